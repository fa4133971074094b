#!/usr/bin/env python
"""Throughput of the batched top-k simplex and top-k cone projections (k = 5) on
N x 1000 float32 rows, 10 % of them with repeated values -- rows/s per job.

One step = one top-k simplex pass plus one top-k cone pass over this rank's
batch (2 * rows projections).  Rows are independent, so ranks shard them with no
data-path collective (weak scaling: every rank owns `--rows` rows).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--rows R]
    python bench.py --impl reference ...   # the reference's CPU path, host cores

`value` is device-resident throughput (CUDA events around K steps, max over
ranks); `e2e` is the same metric through the host-buffer C ABI with the
host<->device copies inside the timed region; `roofline` is the achieved HBM
bandwidth of the slower of the two kernels; `cpu_baseline` is the reference's
own headers timed on a bounded sample on this box's host cores.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = 1000
K_TOP = 5
FULL_ROWS = 262144
BYTES_PER_ROW = 2 * M * 4  # one read + one write of a float32 row
OPS = (("topk_simplex", dict(k=K_TOP, rhs=1.0)), ("topk_cone", dict(k=K_TOP)))

# The other configurations of the benchmark definition, selectable with --config;
# the default (2) is the one the metric is quoted on.
PROX_CONFIGS = {
    1: dict(rows=65536, m=100, dtype="float64", gen="simplex_rows",
            ops=(("knapsack", dict()),),
            name="config 1: simplex projection, 65536 x 100 float64, N(0,1)"),
    3: dict(rows=1048576, m=200, dtype="float32", gen="entropy_rows",
            ops=(("topk_entropy", dict(k=1)), ("topk_entropy", dict(k=10)),
                 ("entropy", dict(hi=1.0, rhs=1.0)), ("lambert_w_exp", dict())),
            name="config 3: top-k entropy k=1,10, entropy, Lambert W(exp x), 1048576 x 200 float32"),
    # Sweeps over the operators of matsdca_prox that the five configurations do not time
    # (include/sdca/prox/*.h): not configurations of the benchmark definition, same shapes and
    # generators as configs 2 and 3 so that the figures sit beside theirs.
    6: dict(rows=131072, m=1000, dtype="float32", gen="topk_rows",
            ops=(("knapsack", dict()), ("knapsack_le", dict()), ("knapsack_le_biased", dict(rho=1.0)),
                 ("topk_simplex", dict(k=K_TOP)), ("topk_simplex_biased", dict(k=K_TOP, rho=1.0)),
                 ("topk_cone", dict(k=K_TOP)), ("topk_cone_biased", dict(k=K_TOP, rho=1.0)),
                 ("two_simplex", dict(p=500)), ("two_simplex_sort", dict(p=500))),
            cpu_rows=16384, no_cpu=("two_simplex_sort",),
            name="operator sweep, Euclidean projections: 131072 x 1000 float32, N(0,1) with ties"),
    7: dict(rows=262144, m=200, dtype="float32", gen="entropy_rows",
            ops=(("entropy", dict(hi=1.0, rhs=1.0)), ("topk_entropy", dict(k=K_TOP)),
                 ("entropy_norm", dict(hi=1.0, rhs=1.0)),
                 ("topk_entropy_biased", dict(k=K_TOP, alpha=1.0))),
            cpu_rows=16384, no_cpu=(),
            name="operator sweep, entropic projections: 262144 x 200 float32, N(0,4)"),
}


# dram__bytes_read.sum + dram__bytes_write.sum of fast_rows_kernel<float,double,top-k simplex,8>
# per row, from the ncu capture summarised in profiles/ (263.1 MB + 209.4 MB over 65536 rows)
NCU_DRAM_BYTES_PER_ROW = 4015 + 3195
# Config 3 (m = 200 float32), same kind of capture on 131072 rows: dram bytes read + written
# per row while the kernel runs (the rest of the 800 B output per row leaves L2 afterwards).
NCU_DRAM_BYTES_PER_ROW_CONFIG3 = {"topk_entropy(k=1)": 801 + 393, "topk_entropy(k=10)": 801 + 390,
                                  "entropy": 801 + 384, "lambert_w_exp": 800 + 479}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()
        self.proc = None

    def run(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            for line in self.proc.stdout:
                self.samples.append(line.strip())
                if self.stop_flag.is_set():
                    break
        except Exception:
            pass

    def finish(self):
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()
        sm, smax, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); smax = max(smax, float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": smax or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def _checker():
    from oracle import refapi
    if refapi.have_reference():
        return refapi.reference(), "reference"
    from oracle import build_oracle
    build_oracle.build_restatement()
    return refapi.restatement(), "port"


def cpu_prox_step(checker, a, work, threads):
    """One step of the workload on the host: both operators, in place on a prepared
    buffer (what matsdca_prox does without an output argument); refilling the buffer
    is outside the timed part.  Returns the timed seconds."""
    dt = 0.0
    for name, kw in OPS:
        np.copyto(work, a)
        t0 = time.perf_counter()
        checker.prox(name, work, nthreads=threads, inplace=True, **kw)
        dt += time.perf_counter() - t0
    return dt


def cpu_baseline(sample_rows, threads, seed):
    """The reference's CPU implementation (its own headers, compiled unmodified)
    on a bounded sample of the same workload."""
    from libsdca_b200 import synth
    checker, kind = _checker()
    a = synth.topk_rows(rows=sample_rows, seed=seed)
    work = np.empty_like(a)
    dt = cpu_prox_step(checker, a, work, threads)
    return {"value": 2 * sample_rows / dt, "unit": "rows/s", "cores": threads, "kind": kind,
            "sample": "%d rows x %d float32 (same generator as the bench), top-k simplex + "
                      "top-k cone, k=5, thresholds in double, in place, rows split over %d host threads"
                      % (sample_rows, M, threads), "seconds": dt}


def run_reference(args, rank, world):
    """`--impl reference`: the reference's own CPU path for the same metric, on the same
    number of rows per step as the GPU arm."""
    if rank != 0:
        return
    from libsdca_b200 import synth
    threads = max(1, min(os.cpu_count() or 1, 64))
    rows = args.rows
    checker, kind = _checker()
    a = synth.topk_rows(rows=rows, seed=2)
    work = np.empty_like(a)
    times = []
    for i in range(args.warmup + args.steps):
        dt = cpu_prox_step(checker, a, work, threads)
        if i >= args.warmup:
            times.append(dt)
    total = sum(times)
    value = 2 * rows * args.steps / total
    base = {"value": value, "unit": "rows/s", "cores": threads, "kind": kind,
            "sample": "every step: %d rows x %d float32 (the GPU arm's rows per GPU), top-k simplex + "
                      "top-k cone, k=5, thresholds in double, in place on a prepared buffer, rows split "
                      "over %d host threads" % (rows, M, threads),
            "seconds": total, "median_step_seconds": float(np.median(times))}
    out = {"impl": "reference", "metric": "prox rows/s (top-k simplex + top-k cone, k=5)",
           "value": value, "unit": "rows/s", "n_gpus": args.gpus, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
           "data": "synthetic",
           "config": workload_config(rows, world, "host arm: one process on this box's cores at every N"),
           "cpu_baseline": base,
           "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0,
                   "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    if not args.no_gap:
        out["gap_eval"] = {"cpu_baseline": gap_cpu_baseline(args, threads)}
    print(json.dumps(out))


def workload_config(rows, world, note):
    return {"workload": "config 2: batched top-k simplex + top-k cone projections, k=5, "
                        "%d x %d float32 per GPU, N(0,1), 10%% rows with tied values" % (rows, M),
            "rows_per_gpu": rows, "m": M, "k": K_TOP, "thresholds_precision": "double",
            "sharding": "rows over %d rank(s), no collective" % world,
            "l2": "inputs (%.2f GB per pass) exceed L2; no flush needed" % (rows * M * 4 / 1e9),
            "note": note}


def _time_op(torch, fn, reps):
    evs = []
    for _ in range(reps):
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    return float(np.median([a.elapsed_time(b) for a, b in evs]))


def other_prox_config(args, rank, world, local_rank):
    """Configs 1 and 3: per-operator device throughput and achieved HBM bandwidth."""
    import torch
    import libsdca_b200 as sd
    from libsdca_b200 import synth
    from oracle import refapi
    cfg = PROX_CONFIGS[args.config]
    torch.cuda.set_device(local_rank)
    rows = cfg["rows"] if args.rows == FULL_ROWS else args.rows
    m = cfg["m"]
    dtype = np.dtype(cfg["dtype"])
    host = getattr(synth, cfg["gen"])(rows=rows)
    a = torch.from_numpy(host).cuda()
    if args.config == 3:
        lam = torch.from_numpy(synth.lambert_inputs(count=rows * m)).cuda().view(rows, m)
    out = torch.empty_like(a)
    peak, peak_kind = measured_peak_gbs()
    bytes_per_row = 2 * m * dtype.itemsize
    per_op = {}
    for name, kw in cfg["ops"]:
        src = lam if name == "lambert_w_exp" else a
        okw = dict(kw) if name == "lambert_w_exp" else dict(kw, precision=args.precision)
        fn = lambda: sd.prox_to(src, out, name, **okw)
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        # inputs smaller than L2 (config 1): rotate over copies so that every launch reads HBM
        if rows * m * dtype.itemsize < (256 << 20):
            copies = [src.clone() for _ in range(8)]
            outs = [torch.empty_like(src) for _ in range(8)]
            it = {"i": 0}

            def fn():
                i = it["i"] = (it["i"] + 1) % 8
                sd.prox_to(copies[i], outs[i], name, **okw)
        ms = _time_op(torch, fn, max(args.steps, 10))
        label = name + ("(k=%d)" % kw["k"] if "k" in kw else "")
        gbs = rows * bytes_per_row / (ms * 1e-3) / 1e9
        per_op[label] = {"ms": ms, "rows_per_s": rows / (ms * 1e-3), "gbs": gbs, "frac": gbs / peak}
    cpu = None
    if not args.no_cpu_baseline and refapi.have_reference():
        threads = max(1, min(os.cpu_count() or 1, 64))
        sample = host[: min(rows, cfg.get("cpu_rows", 65536))]
        cpu = {}
        for name, kw in cfg["ops"]:
            if name in cfg.get("no_cpu", ()):
                # the reference's sort-based walk reads past its arrays on some rows
                # (prox/two_simplex_sort.h:84-97): not run on unchecked rows
                continue
            t0 = time.perf_counter()
            refapi.reference().prox(name, sample, nthreads=threads, **kw)
            label = name + ("(k=%d)" % kw["k"] if "k" in kw else "")
            cpu[label] = {"rows_per_s": len(sample) / (time.perf_counter() - t0), "cores": threads}
    slow = min(per_op, key=lambda k_: per_op[k_]["gbs"])
    total_ms = sum(v["ms"] for v in per_op.values())
    print(json.dumps({
        "metric": "prox rows/s", "value": len(per_op) * rows / (total_ms * 1e-3), "unit": "rows/s",
        "n_gpus": 1, "steps": max(args.steps, 10), "warmup": max(3, args.warmup),
        "ms_per_step": total_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f64" if dtype == np.float64 else "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "rows": rows, "m": m,
                   "thresholds_precision": args.precision,
                   "l2": "rotating buffers" if rows * m * dtype.itemsize < (256 << 20) else "inputs exceed L2"},
        "roofline": {"bound": "hbm", "achieved": per_op[slow]["gbs"], "peak": peak, "unit": "GB/s",
                     "frac": per_op[slow]["frac"],
                     "traffic": (rows * NCU_DRAM_BYTES_PER_ROW_CONFIG3[slow]
                                 if args.config == 3 and m == 200 else None),
                     "kernel": slow,
                     "peak_kind": "of " + peak_kind, "per_operator": per_op},
        "cpu_baseline": cpu, "gpu_launches": len(per_op) * max(args.steps, 10)}))


# dram__bytes_read.sum + dram__bytes_write.sum of one gemm_tf32x3_pair_kernel launch over a chunk of
# 65 536 examples (ncu --set full): 1.360 GB + 0.250 GB; the algorithmic bytes of that chunk are
# 65 536 x (4096 + 1000) x 4 B + 16.4 MB of W = 1.352 GB.  Traffic grows with the examples.
NCU_DRAM_BYTES_PER_EXAMPLE_GAP = (1.360e9 + 0.250e9) / 65536


def gap_roofline(tflops, examples=None):
    """The score GEMM runs on tcgen05 as 3xTF32: three tensor-core products per
    useful multiply-add, TF32 at half the bf16 rate, so the useful-flop ceiling is
    a sixth of the measured bf16 GEMM throughput."""
    peak = None
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            mp = json.load(f)
        bf16 = mp.get("bf16_tflops") or mp.get("bf16_tflops_sustained")   # a kernel timed alone
        peak = float(bf16) / 6.0 if bf16 else None
    except (OSError, ValueError):
        pass
    kind = "of measured" if peak else "of fallback"
    if peak is None:
        peak = 1590.0 / 6.0
    return {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s (useful fp32 flop; 3xTF32)",
            "frac": tflops / peak,
            "traffic": examples * NCU_DRAM_BYTES_PER_EXAMPLE_GAP if examples else None,
            "traffic_note": "dram read + write bytes of the score GEMM for one evaluation on one GPU, scaled by "
                            "examples from the ncu capture of a 65 536-example chunk",
            "peak_kind": kind,
            "kernel": "gemm_tf32x3_pair_kernel (tcgen05 cta_group::2, TMA) + eval_loss_kernel"}


GAP = dict(d=4096, m=1000, k=5, c=1.0, n_total=1048576)
GAP_OBJECTIVES = (("l2_hinge_topk (gamma=0)", 0.0), ("l2_hinge_topk_smooth (gamma=1)", 1.0))
GAP_FIELDS = ("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer", "dual_regularizer")


def gap_problem_device(torch, sd, n, rank):
    """Config 4's data for one rank, generated on the device: class-conditional Gaussian
    blobs (class means ~ N(0, I), noise sigma = 2, labels uniform), and a random feasible
    dual point: v ~ N(0,1)^(m-1) projected onto the top-k simplex, a_j = -v_j, a_y = min(c, sum v)
    -- the form an SDCA step leaves (objective/l2_hinge_topk.h:63-67 of the reference)."""
    d, m, k, c = GAP["d"], GAP["m"], GAP["k"], GAP["c"]
    gen = torch.Generator(device="cuda").manual_seed(5)          # same class means on every rank
    means = torch.randn((m, d), generator=gen, device="cuda")
    gen.manual_seed(50 + rank)
    labels = torch.randint(0, m, (n,), generator=gen, device="cuda")
    X = torch.empty((n, d), device="cuda")
    step_rows = 65536
    for i in range(0, n, step_rows):                                # x_i = mean[y_i] + 2 N(0, I)
        j = min(n, i + step_rows)
        X[i:j] = means[labels[i:j]] + 2.0 * torch.randn((j - i, d), generator=gen, device="cuda")
    v = torch.randn((n, m - 1), generator=gen, device="cuda")
    # rows of 999 floats are not 16-byte aligned: the general kernel handles them
    sd.prox_(v, "topk_simplex", k=k, rhs=c)
    A = torch.zeros((n, m), device="cuda")
    ar = torch.arange(m - 1, device="cuda")[None, :]
    cols = ar + (ar >= labels[:, None])
    A.scatter_(1, cols, -v)
    A[torch.arange(n, device="cuda"), labels] = torch.clamp(v.double().sum(dim=1), max=c).float()
    del v, cols
    return X, labels, A


def gap_problem_host(n, threads):
    """The same family generated on the host with numpy and the reference's own prox, for
    the arm that must not touch the GPU library."""
    d, m, k, c = GAP["d"], GAP["m"], GAP["k"], GAP["c"]
    checker, _ = _checker()
    rng = np.random.default_rng(5)
    means = rng.standard_normal((m, d), dtype=np.float32)
    labels = rng.integers(0, m, n).astype(np.int64)
    X = means[labels] + 2.0 * rng.standard_normal((n, d), dtype=np.float32)
    v = rng.standard_normal((n, m - 1), dtype=np.float32)
    checker.prox("topk_simplex", v, nthreads=threads, inplace=True, k=k, rhs=c)
    A = np.zeros((n, m), dtype=np.float32)
    ar = np.arange(m - 1)[None, :]
    np.put_along_axis(A, ar + (ar >= labels[:, None]), -v, axis=1)
    A[np.arange(n), labels] = np.minimum(c, v.astype(np.float64).sum(axis=1)).astype(np.float32)
    W = np.ascontiguousarray(A.T @ X)                               # d x m column major == (m, d)
    return X, labels, A, W


def gap_cpu_baseline(args, threads, sample=None):
    """The reference's evaluate_dataset (include/sdca/solver/eval.h:15-51: one gemv per
    example, then loss, conjugate and rank) on a contiguous subsample of config 4, examples
    split over the host threads and, for the reference as shipped, on one thread.  The loop
    is linear in the number of examples, so the time for the full 1 048 576 is the sample's
    time scaled by the ratio."""
    from oracle import refapi
    checker, kind = _checker()
    n_s = args.gap_cpu_examples
    if sample is None:
        X, labels, A, W = gap_problem_host(n_s, threads)
    else:
        X, labels, A, W = sample
        n_s = X.shape[0]
    blas = refapi.find_openblas() if kind == "reference" else None
    blas_name = "this repository's sequential CBLAS"
    if blas and checker.use_blas(blas, 1) == 0:
        blas_name = "OpenBLAS from the image, one BLAS thread per host thread"
    kw = dict(W=W, c=GAP["c"], k=GAP["k"])
    t0 = time.perf_counter()
    rec_all = checker.evaluate("l2_hinge_topk", X, A, labels, nthreads=threads, **kw)
    t_all = time.perf_counter() - t0
    n_one = max(1024, n_s // 8)
    t0 = time.perf_counter()
    checker.evaluate("l2_hinge_topk", X[:n_one], A[:n_one], labels[:n_one], nthreads=1, **kw)
    t_one = time.perf_counter() - t0
    if blas:
        checker.use_blas(None, 1)
    scale = GAP["n_total"] / float(n_s)
    return {"value": t_all * scale, "unit": "s per evaluation of 1048576 examples (scaled)",
            "cores": threads, "kind": kind,
            "sample": "evaluate_dataset, top-k hinge alpha k=5 gamma=0, on %d examples of config 4 "
                      "(d=4096, m=1000, float32) split over %d host threads: %.2f s, scaled by %g; "
                      "%s" % (n_s, threads, t_all, scale, blas_name),
            "seconds_sample": t_all,
            "one_thread": {"examples": n_one, "seconds": t_one,
                           "scaled_seconds": t_one * GAP["n_total"] / float(n_one)},
            "record_sample": {f: rec_all[f] for f in GAP_FIELDS}}


def gap_measure(args, rank, world, dist, torch, sd):
    """Seconds per duality-gap evaluation of config 4 (top-k hinge alpha k = 5, features,
    d = 4096, m = 1000, 1 048 576 examples, float32) with the examples sharded over the
    ranks and one all-reduce of the 8 + m sums inside the timed region; the same through
    the host-buffer C ABI; the reference's evaluate_dataset on a subsample beside it."""
    from libsdca_b200 import binding as b
    d, m, k, c, n_total = GAP["d"], GAP["m"], GAP["k"], GAP["c"], GAP["n_total"]
    n = args.gap_examples if args.gap_examples > 0 else n_total // world
    X, labels, A = gap_problem_device(torch, sd, n, rank)
    # W = X A' (d x m, stored (m, d)): the library's eval_recompute_primal, timed as setup
    torch.cuda.synchronize()
    t_primal = time.perf_counter()
    W = sd.primal_from_dual(X, A)
    torch.cuda.synchronize()
    t_primal = time.perf_counter() - t_primal
    torch.cuda.synchronize()
    ws_bytes = sd.lib().sdcab_eval_workspace_bytes
    ws_bytes.restype = C.c_size_t
    workspace = torch.empty(ws_bytes(C.c_int64(n), C.c_int64(m), C.c_int64(4)), dtype=torch.uint8, device="cuda")
    # the library's own communicator (NCCL behind the C ABI): rank 0 makes the id, the
    # process group that torchrun set up only carries it to the other ranks
    comm = None
    if dist is not None:
        ident = [b.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, src=0)
        comm = b.Comm.create(world, rank, ident[0])
        comm.allreduce_(W)                  # the d x m sum of the sharded rebuild W = X A'
        torch.cuda.synchronize()
    reps = max(5, min(args.steps, 10))
    warm = max(3, min(args.warmup, 5))
    results = {}
    for label, gamma in GAP_OBJECTIVES:
        obj = b.make_objective("topk_hinge_alpha", c=c, gamma=gamma, k=k)
        prob = b.make_problem(X, labels, A=A, W=W, include_primal_regularizer=(rank == 0))
        sums = torch.zeros(8 + m, dtype=torch.float64, device="cuda")

        def one_eval():
            if comm is not None:
                comm.eval_sums_(obj, prob, sums, "f32", workspace, workspace.numel())
            else:
                sd.eval_sums_(obj, prob, sums, "f32", workspace, workspace.numel())

        for _ in range(warm):
            one_eval()
        times = []
        for _ in range(reps):
            if dist is not None:
                dist.barrier()
            torch.cuda.synchronize()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); one_eval(); e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            if dist is not None:
                t = torch.tensor([ms], dtype=torch.float64, device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            times.append(ms)
        med = float(np.median(times))
        rec = sd.eval_finish(obj, m, sums.cpu().numpy())
        results[label] = {"seconds_per_eval": med * 1e-3, "best_seconds": min(times) * 1e-3,
                          "evaluations_timed": reps,
                          "tflops": 2.0 * d * m * n * world / (med * 1e-3) / 1e12,
                          "record": {f: rec[f] for f in GAP_FIELDS + ("relative_gap",)},
                          "top1": float(rec["accuracy"][0])}

    # ---- end to end: host buffers through sdcab_eval_f32, each rank its shard, the record
    # terms (sums over the shard's examples) added over the ranks
    obj = b.make_objective("topk_hinge_alpha", c=c, gamma=0.0, k=k)
    hX = torch.empty((n, d), dtype=torch.float32, pin_memory=True)
    hA = torch.empty((n, m), dtype=torch.float32, pin_memory=True)
    hX.copy_(X); hA.copy_(A)
    hW = W.cpu().numpy(); hl = labels.cpu().numpy()
    torch.cuda.synchronize()
    hprob = b.make_problem(hX.numpy(), hl, A=hA.numpy(), W=hW, include_primal_regularizer=(rank == 0))
    rec = b.EvalRecord()
    acc = np.zeros(m)
    fn = sd.lib().sdcab_eval_f32

    def e2e_eval():
        rc = fn(C.byref(obj), C.byref(hprob), C.byref(rec), acc.ctypes.data_as(C.c_void_p))
        if rc != 0:
            raise sd.SdcabError(rc, "sdcab_eval_f32")
        terms = np.array([rec.primal_loss, rec.dual_loss, rec.primal_regularizer, rec.dual_regularizer,
                          acc[0] * n], dtype=np.float64)
        if comm is not None:
            t = torch.from_numpy(terms).cuda()
            comm.allreduce_(t)
            terms = t.cpu().numpy()
        return terms

    e2e_eval()
    e2e_times = []
    terms = None
    for _ in range(max(2, args.e2e_steps)):
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        terms = e2e_eval()
        dt = time.perf_counter() - t0
        if dist is not None:
            t = torch.tensor([dt], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e_times.append(dt)
    e2e_s = float(np.median(e2e_times))
    first = results[GAP_OBJECTIVES[0][0]]
    dev_rec = first["record"]
    e2e = {"seconds_per_eval": e2e_s, "evaluations_timed": len(e2e_times),
           "h2d_bytes_per_eval": (n * d * 4 + n * m * 4 + n * 8) * world + d * m * 4 * world,
           "d2h_bytes_per_eval": (8 + m) * 8 * world,
           "pcie_gbs_per_rank": (n * d * 4 + n * m * 4) / e2e_s / 1e9,
           "record_vs_device": {
               "primal_loss": abs(terms[0] - dev_rec["primal_loss"]) / max(1.0, abs(dev_rec["primal_loss"])),
               "dual_loss": abs(terms[1] - dev_rec["dual_loss"]) / max(1.0, abs(dev_rec["dual_loss"])),
               "primal_regularizer": abs(terms[2] - dev_rec["primal_regularizer"]) / max(1.0, abs(dev_rec["primal_regularizer"])),
               "top1": abs(terms[4] / (n * world) - first["top1"])}}
    del hX, hA

    # ---- the reference on a subsample of rank 0's shard, every term compared with the
    # device evaluation of the same examples
    cpu = None
    parity = None
    if rank == 0 and not args.no_cpu_baseline:
        n_s = min(n, args.gap_cpu_examples)
        Xs, As, ls = X[:n_s].contiguous(), A[:n_s].contiguous(), labels[:n_s].contiguous()
        Ws = sd.primal_from_dual(Xs, As)        # the sample's own W, so that its gap is a real gap
        sample = (Xs.cpu().numpy(), ls.cpu().numpy(), As.cpu().numpy(), Ws.cpu().numpy())
        threads = max(1, min(os.cpu_count() or 1, 64))
        cpu = gap_cpu_baseline(args, threads, sample)
        dev = sd.evaluate(b.make_objective("topk_hinge_alpha", c=c, gamma=0.0, k=k), Xs, ls, A=As, W=Ws)
        ref_rec = cpu["record_sample"]
        exact_reg = 0.5 * float((sample[3].astype(np.float64) ** 2).sum())
        parity = {f: abs(dev[f] - ref_rec[f]) / max(1.0, abs(ref_rec[f])) for f in GAP_FIELDS}
        # the same examples with the dual point scaled down until the margins are of order
        # one and some are violated (at the benchmark's own dual point every primal loss is 0)
        s2 = 0.5 / (n_s / 1000.0 * 4096.0 + 2.0e4)
        As2 = (As * s2).contiguous()
        Ws2 = sd.primal_from_dual(Xs, As2)
        checker, _ = _checker()
        parity_scaled = {}
        for label, gamma in GAP_OBJECTIVES:
            name = "l2_hinge_topk" if gamma == 0.0 else "l2_hinge_topk_smooth"
            r2 = checker.evaluate(name, sample[0], As2.cpu().numpy(), sample[1], W=Ws2.cpu().numpy(),
                                  c=c, gamma=gamma, k=k, nthreads=threads)
            d2 = sd.evaluate(b.make_objective("topk_hinge_alpha", c=c, gamma=gamma, k=k), Xs, ls, A=As2, W=Ws2)
            parity_scaled[label] = {
                "reference_primal_loss": r2["primal_loss"], "reference_dual_loss": r2["dual_loss"],
                "primal_loss": abs(d2["primal_loss"] - r2["primal_loss"]) / max(1.0, abs(r2["primal_loss"])),
                "dual_loss": abs(d2["dual_loss"] - r2["dual_loss"]) / max(1.0, abs(r2["dual_loss"])),
                "accuracy_max_abs": float(np.abs(d2["accuracy"] - r2["accuracy"]).max())}
        parity["scaled_dual_point"] = parity_scaled
        parity["note"] = ("relative to max(1, |reference|) on %d examples; the reference sums 0.5 ||W||^2 "
                          "over 4.1e6 float32 terms in float, this library in double: the regulariser "
                          "terms (and primal / dual, which contain them) differ by the reference's own "
                          "rounding; against the exact double value this library is at %.1e"
                          % (n_s, abs(dev["primal_regularizer"] - exact_reg) / exact_reg))
    out = {"workload": "config 4: duality-gap evaluation, top-k hinge alpha k=5, features d=%d, m=%d, "
                       "%d examples in total, float32" % (d, m, n * world),
           "examples_per_gpu": n, "n_gpus": world,
           "scaling": "strong" if args.gap_examples <= 0 else "weak",
           "collective": "one ncclAllReduce(sum) of %d doubles per evaluation through the library's "
                         "communicator (sdcab_eval_sums_sharded_f32_dev), inside the timed region" % (8 + m),
           "timing": "CUDA events around each evaluation, median of %d, max over ranks" % reps,
           "seconds_per_eval": first["seconds_per_eval"],
           "results": results, "roofline": gap_roofline(first["tflops"] / world, n),
           "e2e": e2e, "cpu_baseline": cpu, "parity_on_sample": parity,
           "setup_primal_from_dual": {"seconds": t_primal, "tflops": 2.0 * d * m * n / t_primal / 1e12}}
    if comm is not None:
        torch.cuda.synchronize()
        comm.destroy()
    del X, A, W, workspace
    torch.cuda.empty_cache()
    return out


def gap_config(args, rank, world, local_rank):
    """Config 4 on its own (`--config 4`): the gap evaluation as the line's metric."""
    import torch
    import libsdca_b200 as sd
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.rows != FULL_ROWS and args.gap_examples <= 0:
        args.gap_examples = args.rows
    g = gap_measure(args, rank, world, dist, torch, sd)
    if rank == 0:
        first = g["results"][GAP_OBJECTIVES[0][0]]
        print(json.dumps({
            "metric": "duality-gap evaluation seconds", "value": first["seconds_per_eval"], "unit": "s",
            "n_gpus": world, "steps": first["evaluations_timed"], "warmup": 3,
            "ms_per_step": first["seconds_per_eval"] * 1e3, "higher_is_better": False,
            "scaling": g["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": g["workload"], "examples_per_gpu": g["examples_per_gpu"],
                       "collective": g["collective"]},
            "roofline": g["roofline"], "cpu_baseline": g["cpu_baseline"],
            "e2e": {"value": g["e2e"]["seconds_per_eval"], "unit": "s",
                    "h2d_bytes_per_step": g["e2e"]["h2d_bytes_per_eval"],
                    "d2h_bytes_per_step": g["e2e"]["d2h_bytes_per_eval"]},
            "gpu_launches": 8 * first["evaluations_timed"] * world,
            "gap_eval": g}))
    if dist is not None:
        dist.destroy_process_group()


def rbf_problem(torch, n, seed=6, dim=128, m=100, sigma=1.5):
    """Config 5's data on the device: Gaussian blobs and their RBF Gram matrix,
    gamma = 1 / dim, float64 (the same construction as synth.kernel_problem)."""
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    means = torch.randn(m, dim, generator=g, device="cuda", dtype=torch.float64)
    labels = torch.randint(0, m, (n,), generator=g, device="cuda")
    P = means[labels] + sigma * torch.randn(n, dim, generator=g, device="cuda", dtype=torch.float64)
    sq = (P * P).sum(1)
    K = P @ P.T
    K.mul_(-2).add_(sq[:, None]).add_(sq[None, :]).clamp_(min=0).div_(-dim).exp_()
    return K, labels


def fit_config(args, rank, world, local_rank):
    """Config 5: Crammer-Singer SDCA fit, kernel input, N = 50000 (or --rows),
    m = 100, float64, epsilon = 1e-3, gap evaluated every epoch.  The steps of an
    epoch are sequential, so ranks do not share the work: every rank runs the
    same fit (replicas only) and rank 0 reports."""
    import torch
    import libsdca_b200 as sd
    torch.cuda.set_device(local_rank)
    n = args.rows if args.rows != FULL_ROWS else 50000
    m = 100
    K, labels = rbf_problem(torch, n)
    A = torch.zeros(n, m, device="cuda", dtype=torch.float64)
    # warm-up on a small problem (module load, workspace growth)
    Kw, lw = rbf_problem(torch, 2048, seed=7)
    sd.fit_(4, Kw, lw, torch.zeros(2048, m, device="cuda", dtype=torch.float64), kernel=True,
            c=1.0, k=1, max_epoch=3, eval_epoch=1)
    del Kw, lw
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    t0 = time.perf_counter()
    r = sd.fit_(4, K, labels, A, kernel=True, c=1.0, k=1, max_epoch=args.max_epoch, eval_epoch=1,
                epsilon=1e-3)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clocks = sampler.finish() if sampler else None
    if rank != 0:
        return
    epochs = max(1, r["epoch"])
    last = r["history"][-1]
    out = {
        "metric": "SDCA fit seconds per epoch (Crammer-Singer, kernel input, gap evaluated every epoch)",
        "value": (r["solve_seconds"] + r["eval_seconds"]) / epochs, "unit": "s", "n_gpus": world,
        "steps": epochs, "warmup": 1, "ms_per_step": 1e3 * (r["solve_seconds"] + r["eval_seconds"]) / epochs,
        "higher_is_better": False, "scaling": "replicas only", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": "config 5: msvm (l2_topk_hinge, k=1, c=1) fit on an RBF Gram matrix, "
                               "N=%d, m=100, float64, epsilon=1e-3, eval_epoch=1" % n, "examples": n},
        "fit": {"status": r["status"], "epochs": r["epoch"], "solve_seconds": r["solve_seconds"],
                "eval_seconds": r["eval_seconds"], "seconds_per_epoch_updates": r["solve_seconds"] / epochs,
                "seconds_per_evaluation": r["eval_seconds"] / max(1, r["num_evals"]),
                "wall_seconds": wall, "primal": last["primal"], "dual": last["dual"],
                "relative_gap": last["relative_gap"]},
        "roofline": {"bound": "latency (a chain of N dependent steps per epoch)",
                     "achieved": 1e6 * r["solve_seconds"] / epochs / n, "peak": None,
                     "unit": "us/step", "frac": None, "traffic": None,
                     "kernel": "fit_chain_kernel + gemm_kernel<double,64,128,8,8,4> (mma.sync f64)"},
        "gpu_launches": int(3 * ((n + 63) // 64) * r["epoch"] + 6 * r["num_evals"]),
        "clocks": clocks,
    }
    if not args.no_cpu_baseline:
        out["cpu_baseline"] = fit_cpu_baseline(args.cpu_fit_examples, sd, torch)
    print(json.dumps(out))


FIT_SWEEP = (("l2_topk_hinge", 4, False), ("l2_topk_hinge_smooth", 5, False), ("l2_hinge_topk", 2, False),
             ("l2_hinge_topk_smooth", 3, False), ("l2_entropy", 0, False), ("l2_entropy_topk", 1, False),
             ("l2_multilabel_hinge", 6, True), ("l2_multilabel_hinge_smooth", 7, True),
             ("l2_multilabel_entropy", 8, True))


def fit_sweep_config(args, rank, world, local_rank):
    """`--config 8`: the update steps of all nine objectives (update_dual_variables of
    include/sdca/solver/objective/*.h), not a configuration of the benchmark definition:
    three epochs of each on class-conditional Gaussian blobs, N = 16384 (or --rows), m = 100,
    float64, as a Gram matrix (kernel input) and as d = 256 features; microseconds per step
    from the device time of the update steps, the reference's solver on 2048 examples beside it."""
    import torch
    import libsdca_b200 as sd
    from oracle import refapi
    if rank != 0:
        return
    torch.cuda.set_device(local_rank)
    n = args.rows if args.rows != FULL_ROWS else 16384
    m, d, k, epochs = 100, 256, 3, 3
    rng = np.random.default_rng(11)
    means = rng.standard_normal((m, d))
    labels = rng.integers(0, m, n).astype(np.int64)
    X = (means[labels] + 1.5 * rng.standard_normal((n, d))) / np.sqrt(d)
    extra = rng.integers(0, m, (n, 2))
    ml_lists = [sorted(set([int(labels[i])] + [int(e) for e in extra[i][: int(rng.integers(0, 3))]])) for i in range(n)]
    ml_labels = np.array([c_ for l in ml_lists for c_ in l], dtype=np.int64)
    ml_offsets = np.concatenate([[0], np.cumsum([len(l) for l in ml_lists])]).astype(np.int64)
    tX = torch.from_numpy(X).cuda()
    tK = tX @ tX.T
    have_ref = (not args.no_cpu_baseline) and refapi.have_reference()
    n_ref = min(n, 2048)
    per = {}
    for name, oid, ml in FIT_SWEEP:
        lab = torch.from_numpy(ml_labels if ml else labels).cuda()
        off = torch.from_numpy(ml_offsets).cuda() if ml else None
        row = {}
        for kernel in (True, False):
            A = torch.zeros(n, m, device="cuda", dtype=torch.float64)
            W = None if kernel else torch.zeros(m, d, device="cuda", dtype=torch.float64)
            r = sd.fit_(oid, tK if kernel else tX, lab, A, W=W, kernel=kernel, offsets=off, c=1.0, gamma=1.0,
                        k=k, max_epoch=epochs, eval_epoch=epochs, epsilon=1e-12)
            torch.cuda.synchronize()
            last = r["history"][-1]
            row["kernel" if kernel else "features"] = {
                "us_per_step": 1e6 * r["solve_seconds"] / (n * max(1, r["epoch"])), "epochs": r["epoch"],
                "seconds_per_evaluation": r["eval_seconds"] / max(1, r["num_evals"]),
                "relative_gap": last["relative_gap"], "status": r["status"]}
        if have_ref:
            nl = ml_offsets[n_ref]
            A_ref = np.zeros((n_ref, m)); W_ref = np.zeros((m, d))
            t0 = time.perf_counter()
            rr = refapi.reference().fit(name, X[:n_ref], A_ref, (ml_labels[:nl] if ml else labels[:n_ref]), W=W_ref,
                                        offsets=(ml_offsets[: n_ref + 1] if ml else None), c=1.0, gamma=1.0, k=k,
                                        max_epoch=epochs, eval_epoch=epochs, epsilon=1e-12)
            dt = time.perf_counter() - t0
            row["reference_features"] = {"us_per_step": 1e6 * dt / (n_ref * max(1, rr["epoch"])), "examples": n_ref,
                                         "cores": 1, "note": "whole call including its one evaluation"}
        per[name] = row
    slow = max(per, key=lambda q: per[q]["kernel"]["us_per_step"])
    print(json.dumps({
        "metric": "SDCA update microseconds per step, all objectives", "value": per[slow]["kernel"]["us_per_step"],
        "unit": "us/step", "n_gpus": 1, "steps": epochs, "warmup": 0, "ms_per_step": None,
        "higher_is_better": False, "scaling": "replicas only", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": "fit sweep: %d examples, m=%d, d=%d, k=%d, c=1, gamma=1, float64, %d epochs per "
                               "objective, kernel and feature input" % (n, m, d, k, epochs)},
        "roofline": {"bound": "latency (a chain of dependent steps)", "achieved": per[slow]["kernel"]["us_per_step"],
                     "peak": None, "unit": "us/step", "frac": None, "traffic": None, "kernel": slow,
                     "per_objective": per},
        "gpu_launches": None}))


def fit_cpu_baseline(n_small, sd, torch):
    """The reference's solver on a bounded problem of the same family (the full size
    would take it hours: an epoch reads A once per example, N^2 m multiply-adds), and
    the same problem through the device fit for the comparison of the results."""
    from libsdca_b200 import synth
    from oracle import refapi
    if refapi.have_reference():
        ref, kind = refapi.reference(), "reference"
    else:
        from oracle import build_oracle
        build_oracle.build_restatement()
        ref, kind = refapi.restatement(), "port"
    K, labels = synth.kernel_problem(n=n_small, seed=6)
    A_ref = np.zeros((n_small, 100))
    t0 = time.perf_counter()
    r = ref.fit("l2_topk_hinge", K, A_ref, labels, kernel=True, c=1.0, k=1, epsilon=1e-3,
                max_epoch=200, eval_epoch=1)
    dt = time.perf_counter() - t0
    A = torch.zeros(n_small, 100, device="cuda", dtype=torch.float64)
    g = sd.fit_(4, torch.from_numpy(K).cuda(), torch.from_numpy(labels).cuda(), A, kernel=True, c=1.0,
                k=1, epsilon=1e-3, max_epoch=200, eval_epoch=1)
    return {"value": dt / max(1, r["epoch"]), "unit": "s/epoch", "cores": 1, "kind": kind,
            "sample": "the reference's solver::solve (sequential BLAS) on N=%d of the same generator, "
                      "%d epochs to epsilon=1e-3; its epoch cost grows with N^2" % (n_small, r["epoch"]),
            "seconds": dt, "epochs": r["epoch"],
            "device_same_problem": {"epochs": g["epoch"], "status": g["status"],
                                    "seconds": g["solve_seconds"] + g["eval_seconds"],
                                    "max_abs_diff_A": float(np.abs(A.cpu().numpy() - A_ref).max()),
                                    "primal_diff": abs(g["history"][-1]["primal"] - r["history"][-1][0]),
                                    "dual_diff": abs(g["history"][-1]["dual"] - r["history"][-1][1])}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--rows", type=int, default=FULL_ROWS, help="rows per GPU")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-rows", type=int, default=65536, help="rows of the CPU sample")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--max-epoch", type=int, default=100, help="config 5: epoch limit")
    ap.add_argument("--cpu-fit-examples", type=int, default=4000,
                    help="config 5: size of the problem the reference's solver is timed on")
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 4, 5, 6, 7, 8],
                    help="benchmark configuration; 2 (default) is the headline")
    ap.add_argument("--no-gap", action="store_true",
                    help="leave the duality-gap evaluation (config 4) out of the default line")
    ap.add_argument("--gap-examples", type=int, default=0,
                    help="config 4: examples per GPU (default: 1048576 / N, strong scaling)")
    ap.add_argument("--gap-cpu-examples", type=int, default=65536,
                    help="config 4: examples of the subsample the reference's evaluate_dataset is timed on")
    ap.add_argument("--regions", type=int, default=5,
                    help="timed regions of --steps steps each; the median region is reported")
    ap.add_argument("--precision", default="double", choices=["double", "float"],
                    help="precision of thresholds and accumulators")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.config in PROX_CONFIGS:
        return other_prox_config(args, rank, world, local_rank)
    if args.config == 4:
        return gap_config(args, rank, world, local_rank)
    if args.config == 8:
        return fit_sweep_config(args, rank, world, local_rank)
    if args.config == 5:
        return fit_config(args, rank, world, local_rank)

    import torch
    import libsdca_b200 as sd
    from libsdca_b200 import synth

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    warmup = max(args.warmup, 3)
    rows = args.rows
    host = synth.topk_rows(rows=rows, seed=2 + rank)
    pinned_in = torch.from_numpy(host).pin_memory()
    pinned_out = torch.empty_like(pinned_in).pin_memory()
    a = pinned_in.cuda(non_blocking=True)
    out = torch.empty_like(a)
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def step():
        for name, kw in OPS:
            sd.prox_to(a, out, name, precision=args.precision, **kw)

    for _ in range(warmup):
        step()
    barrier()

    # per-kernel durations (CUDA events on the launching stream) for the roofline
    per_op_ms = {}
    for name, kw in OPS:
        evs = []
        for _ in range(max(3, min(args.steps, 10))):
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); sd.prox_to(a, out, name, precision=args.precision, **kw); e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        per_op_ms[name] = float(np.mean([x.elapsed_time(y) for x, y in evs]))

    # the same kernels with float thresholds (opts.precision = 'single'), for reference
    other = "float" if args.precision == "double" else "double"
    per_op_other = {}
    for name, kw in OPS:
        per_op_other[name] = _time_op(torch, lambda: sd.prox_to(a, out, name, precision=other, **kw), 5)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()

    def keep_busy(samples_wanted, limit_s):
        # untimed steps until nvidia-smi has delivered its samples: they are taken while
        # the kernels of the timed region run (the region itself lasts a few milliseconds)
        t0 = time.perf_counter()
        while sampler and len(sampler.samples) < samples_wanted and time.perf_counter() - t0 < limit_s:
            step()
            torch.cuda.synchronize()

    keep_busy(2, 3.0)
    # the W untimed warm-up steps run again here, so that the timed region starts on a busy GPU
    for _ in range(warmup):
        step()
    # `--regions` timed regions of exactly `--steps` steps each, every one bracketed by a
    # barrier and a device synchronisation; the median region is the one reported (a single
    # region of a few milliseconds reads a few per cent off from run to run)
    region_ms = []
    for _ in range(max(1, args.regions)):
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        region_ms.append(max_over_ranks(e0.elapsed_time(e1)))
    elapsed_ms = float(np.median(region_ms))
    keep_busy(4, 1.5)
    clocks = sampler.finish() if sampler else None

    # end to end through the host-buffer C ABI: pinned host in, pinned host out
    lib = sd.lib()
    from libsdca_b200.binding import make_opts

    def e2e_step():
        for name, kw in OPS:
            o = make_opts(precision=args.precision, **kw)
            rc = lib.sdcab_prox_f32(name.encode(), C.c_void_p(pinned_in.data_ptr()), C.c_int64(M),
                                    C.c_int64(rows), C.byref(o), C.c_void_p(pinned_out.data_ptr()))
            if rc != 0:
                raise sd.SdcabError(rc, "sdcab_prox_f32")

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e_step()
    own_e2e_s = time.perf_counter() - t0
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    checksum = float(pinned_out[:: max(1, rows // 64)].double().sum())
    # per-rank PCIe rate of the host-buffer path (both directions run at once): slowest rank
    pcie_gbs = -max_over_ranks(-(2 * rows * M * 4 * args.e2e_steps) / own_e2e_s / 1e9)
    # what the platform gives the same buffers with no kernel in between: every rank copies its
    # pinned input to the device and a device buffer to its pinned output at the same time
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def plain_copies():
        with torch.cuda.stream(s_in):
            a.copy_(pinned_in, non_blocking=True)
        with torch.cuda.stream(s_out):
            pinned_out.copy_(out, non_blocking=True)
        s_in.synchronize(); s_out.synchronize()

    plain_copies()
    barrier()
    t0 = time.perf_counter()
    for _ in range(3):
        plain_copies()
    own_copy_s = (time.perf_counter() - t0) / 3
    barrier()
    copy_gbs = -max_over_ranks(-(rows * M * 4) / own_copy_s / 1e9)
    del pinned_in, pinned_out, a, out
    torch.cuda.empty_cache()
    sd.lib().sdcab_release_workspace()

    gap = None
    if not args.no_gap:
        gap = gap_measure(args, rank, world, dist, torch, sd)

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        slow = max(per_op_ms, key=per_op_ms.get)
        achieved = rows * BYTES_PER_ROW / (per_op_ms[slow] * 1e-3) / 1e9
        value = 2.0 * rows * world * args.steps / (elapsed_ms * 1e-3)
        result = {
            "metric": "prox rows/s (top-k simplex + top-k cone, k=5)",
            "value": value, "unit": "rows/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(rows, world, "device-resident inputs, out-of-place kernels"),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": rows * NCU_DRAM_BYTES_PER_ROW, "kernel": slow,
                         "traffic_note": "dram read + write bytes of one launch, scaled by rows from the ncu "
                                         "capture of a 65536-row launch (4015 B read + 3195 B written per row "
                                         "while the kernel runs; the last 805 B per row leave L2 afterwards; the "
                                         "row's second read is served by L2)",
                         "peak_kind": "of " + peak_kind,
                         "per_kernel_ms": per_op_ms,
                         "per_kernel_gbs": {k: rows * BYTES_PER_ROW / (v * 1e-3) / 1e9
                                            for k, v in per_op_ms.items()},
                         "thresholds_precision": args.precision,
                         "per_kernel_gbs_%s_thresholds" % other:
                             {k: rows * BYTES_PER_ROW / (v * 1e-3) / 1e9 for k, v in per_op_other.items()}},
            "e2e": {"value": 2.0 * rows * world * args.e2e_steps / e2e_s, "unit": "rows/s",
                    "h2d_bytes_per_step": 2 * rows * M * 4 * world, "d2h_bytes_per_step": 2 * rows * M * 4 * world,
                    "steps": args.e2e_steps, "checksum": checksum,
                    "pcie_gbs_each_way_slowest_rank": pcie_gbs,
                    "plain_copy_gbs_each_way_slowest_rank": copy_gbs,
                    "note": "the second figure is the same pinned buffers copied both ways at once by "
                            "every rank with no kernel in between: the host side's ceiling for this path"},
            "gpu_launches": 2 * args.steps * world * max(1, args.regions),
            "timed_regions_ms": region_ms,
            "clocks": clocks,
        }
        result["config"]["timing"] = ("%d regions of %d steps, each bracketed by barrier + synchronize; "
                                      "value and ms_per_step are the median region's" % (len(region_ms), args.steps))
        if gap is not None:
            result["gap_eval"] = gap
        if not args.no_cpu_baseline and world == 1:
            threads = max(1, min(os.cpu_count() or 1, 64))
            result["cpu_baseline"] = cpu_baseline(args.cpu_rows, threads, seed=2)
        print(json.dumps(result))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
