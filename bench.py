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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

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
            sd.prox_to(a, out, name, **kw)

    for _ in range(warmup):
        step()
    barrier()

    # per-kernel durations (CUDA events on the launching stream) for the roofline
    per_op_ms = {}
    for name, kw in OPS:
        evs = []
        for _ in range(max(3, min(args.steps, 10))):
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); sd.prox_to(a, out, name, **kw); e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        per_op_ms[name] = float(np.mean([x.elapsed_time(y) for x, y in evs]))

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed_ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.finish() if sampler else None

    # end to end through the host-buffer C ABI: pinned host in, pinned host out
    lib = sd.lib()
    from libsdca_b200.binding import make_opts

    def e2e_step():
        for name, kw in OPS:
            o = make_opts(**kw)
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
                         "frac": achieved / peak, "traffic": None, "kernel": slow,
                         "peak_kind": "of " + peak_kind,
                         "per_kernel_ms": per_op_ms,
                         "per_kernel_gbs": {k: rows * BYTES_PER_ROW / (v * 1e-3) / 1e9
                                            for k, v in per_op_ms.items()}},
            "e2e": {"value": 2.0 * rows * world * args.e2e_steps / e2e_s, "unit": "rows/s",
                    "h2d_bytes_per_step": 2 * rows * M * 4, "d2h_bytes_per_step": 2 * rows * M * 4,
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
