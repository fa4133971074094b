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


def cpu_baseline(sample_rows, threads, seed):
    """The reference's CPU implementation (its own headers, compiled unmodified)
    on a bounded sample of the same workload."""
    from libsdca_b200 import synth
    from oracle import refapi
    if refapi.have_reference():
        checker, kind = refapi.reference(), "reference"
    else:
        from oracle import build_oracle
        build_oracle.build_restatement()
        checker, kind = refapi.restatement(), "port"
    a = synth.topk_rows(rows=sample_rows, seed=seed)
    t0 = time.perf_counter()
    for name, kw in OPS:
        checker.prox(name, a, nthreads=threads, **kw)
    dt = time.perf_counter() - t0
    return {"value": 2 * sample_rows / dt, "unit": "rows/s", "cores": threads, "kind": kind,
            "sample": "%d rows x %d float32 (same generator as the bench), top-k simplex + "
                      "top-k cone, k=5, thresholds in double, rows split over %d host threads"
                      % (sample_rows, M, threads), "seconds": dt}


def run_reference(args, rank, world):
    """`--impl reference`: the reference's own CPU path for the same metric."""
    if rank != 0:
        return
    threads = max(1, min(os.cpu_count() or 1, 64))
    sample_rows = args.cpu_rows
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(sample_rows, threads, seed=2)
        if i >= args.warmup:
            times.append(base["seconds"])
    total = sum(times)
    value = 2 * sample_rows * args.steps / total
    base["value"] = value
    out = {"impl": "reference", "metric": "prox rows/s (top-k simplex + top-k cone, k=5)",
           "value": value, "unit": "rows/s", "n_gpus": args.gpus, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
           "data": "synthetic", "config": workload_config(sample_rows, world, "bounded sample per step"),
           "cpu_baseline": base,
           "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0,
                   "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
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
        sample = host[: min(rows, 65536)]
        cpu = {}
        for name, kw in cfg["ops"]:
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


def gap_roofline(tflops):
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
            "frac": tflops / peak, "traffic": None, "peak_kind": kind,
            "kernel": "gemm_tf32x3_kernel (tcgen05, TMA) + eval_loss_kernel"}


def gap_config(args, rank, world, local_rank):
    """Config 4: duality-gap evaluation, top-k hinge alpha (k = 5), feature input,
    d = 4096, m = 1000, float32; examples sharded over the ranks, one all-reduce
    of the sums vector.  --rows sets the examples per GPU (default 1048576 / N)."""
    import torch
    import libsdca_b200 as sd
    from libsdca_b200 import binding as b
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    d, m, k, c = 4096, 1000, 5, 1.0
    n_total = 1048576
    n = args.rows if args.rows != FULL_ROWS else n_total // world
    gen = torch.Generator(device="cuda").manual_seed(5)          # same class means on every rank
    means = torch.randn((m, d), generator=gen, device="cuda")
    gen.manual_seed(50 + rank)
    labels = torch.randint(0, m, (n,), generator=gen, device="cuda")
    X = torch.empty((n, d), device="cuda")
    step_rows = 65536
    for i in range(0, n, step_rows):                                # x_i = mean[y_i] + 2 N(0, I)
        j = min(n, i + step_rows)
        X[i:j] = means[labels[i:j]] + 2.0 * torch.randn((j - i, d), generator=gen, device="cuda")
    # a random feasible dual point: v ~ N(0,1)^(m-1) projected onto the top-k simplex
    v = torch.randn((n, m - 1), generator=gen, device="cuda")
    # rows of 999 floats are not 16-byte aligned: the general kernel handles them
    sd.prox_(v, "topk_simplex", k=k, rhs=c)
    A = torch.zeros((n, m), device="cuda")
    cols = torch.arange(m - 1, device="cuda")[None, :] + (torch.arange(m - 1, device="cuda")[None, :] >= labels[:, None])
    A.scatter_(1, cols, -v)
    A[torch.arange(n, device="cuda"), labels] = torch.clamp(v.double().sum(dim=1), max=c).float()
    del v, cols
    # W = X A' (d x m, stored (m, d)): the library's eval_recompute_primal, timed as setup
    torch.cuda.synchronize()
    t_primal = time.perf_counter()
    W = sd.primal_from_dual(X, A)
    torch.cuda.synchronize()
    t_primal = time.perf_counter() - t_primal
    if dist is not None:
        dist.all_reduce(W)
    torch.cuda.synchronize()
    results = {}
    ws_bytes = sd.lib().sdcab_eval_workspace_bytes
    ws_bytes.restype = C.c_size_t
    workspace = torch.empty(ws_bytes(C.c_int64(n), C.c_int64(m), C.c_int64(4)), dtype=torch.uint8, device="cuda")
    for label, gamma in (("l2_hinge_topk (gamma=0)", 0.0), ("l2_hinge_topk_smooth (gamma=1)", 1.0)):
        obj = b.make_objective("topk_hinge_alpha", c=c, gamma=gamma, k=k)
        prob = b.make_problem(X, labels, A=A, W=W, include_primal_regularizer=(rank == 0))
        sums = torch.zeros(8 + m, dtype=torch.float64, device="cuda")

        def one_eval():
            sd.eval_sums_(obj, prob, sums, "f32", workspace, workspace.numel())
            if dist is not None:
                dist.all_reduce(sums)
            return sums

        for _ in range(max(1, min(args.warmup, 3))):
            one_eval()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        steps = max(1, min(args.steps, 5))
        e0.record()
        for _ in range(steps):
            one_eval()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        if dist is not None:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        rec = sd.eval_finish(obj, m, sums.cpu().numpy())
        results[label] = {"seconds_per_eval": ms * 1e-3,
                          "tflops": 2.0 * d * m * n * world / (ms * 1e-3) / 1e12,
                          "record": {f: rec[f] for f in ("primal", "dual", "primal_loss", "dual_loss",
                                                         "primal_regularizer", "relative_gap")},
                          "top1": float(rec["accuracy"][0])}
    if rank == 0:
        first = results["l2_hinge_topk (gamma=0)"]
        print(json.dumps({
            "metric": "duality-gap evaluation seconds", "value": first["seconds_per_eval"], "unit": "s",
            "n_gpus": world, "steps": max(1, min(args.steps, 5)), "warmup": max(1, min(args.warmup, 3)),
            "ms_per_step": first["seconds_per_eval"] * 1e3, "higher_is_better": False,
            "scaling": "strong" if args.rows == FULL_ROWS else "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "config 4: gap evaluation, top-k hinge alpha k=5, features d=4096, m=1000, "
                                   "%d examples per GPU, float32" % n, "examples_per_gpu": n,
                       "collective": "one all_reduce(sum) of %d doubles" % (8 + m),
                       "setup_primal_from_dual": {"seconds": t_primal,
                                                  "tflops": 2.0 * d * m * n / t_primal / 1e12}},
            "roofline": gap_roofline(first["tflops"]),
            "results": results}))
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
                     "kernel": "fit_chain_kernel + gemm_kernel<double,64,64,8,4,4>"},
        "gpu_launches": int(3 * ((n + 63) // 64) * r["epoch"] + 6 * r["num_evals"]),
        "clocks": clocks,
    }
    if not args.no_cpu_baseline:
        out["cpu_baseline"] = fit_cpu_baseline(args.cpu_fit_examples, sd, torch)
    print(json.dumps(out))


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
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 4, 5],
                    help="benchmark configuration; 2 (default) is the headline")
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
    barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed_ms = max_over_ranks(e0.elapsed_time(e1))
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
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    checksum = float(pinned_out[:: max(1, rows // 64)].double().sum())

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
                    "steps": args.e2e_steps, "checksum": checksum},
            "gpu_launches": 2 * args.steps * world,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            threads = max(1, min(os.cpu_count() or 1, 64))
            result["cpu_baseline"] = cpu_baseline(args.cpu_rows, threads, seed=2)
        print(json.dumps(result))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
