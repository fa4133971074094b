"""Host side of the sharded gap evaluation on CPU ranks (gloo, world size 2):
each rank produces the sums of its shard, one all-reduce adds them, and
eval_finish on the reduced vector equals the unsharded record.  The per-shard
sums come from the host-lane build of the loss code (no GPU here); the recipe
is the one the benchmark uses with NCCL."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, kernel, out_dir):
    sys.path.insert(0, ROOT)
    import ctypes as C
    import torch
    import torch.distributed as dist
    from libsdca_b200 import binding as b
    from tests.hostsim import build as hb
    from tests.test_oracle_restatement import random_problem
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sim = hb.load()
    rng = np.random.default_rng(5)
    n, d, m = 60, 10, 8
    X, labels, _ = random_problem(rng, n, d, m, np.float64, False)
    A = -np.abs(rng.standard_normal((n, m))) * 0.01
    A[np.arange(n), labels] = 0.04
    W = rng.standard_normal((m, d))
    K = X @ X.T
    obj = b.make_objective(5, c=1.0, gamma=0.5, k=1)
    lo, hi = n * rank // world, n * (rank + 1) // world
    if kernel:
        prob = b.make_problem(np.ascontiguousarray(K[lo:hi]), np.ascontiguousarray(labels[lo:hi]),
                              A=A, kernel=True, a_row_offset=lo)
    else:
        prob = b.make_problem(np.ascontiguousarray(X[lo:hi]), np.ascontiguousarray(labels[lo:hi]),
                              A=A, W=W, a_row_offset=lo, include_primal_regularizer=(rank == 0))
    sums = np.zeros(8 + m)
    assert sim.lib.sdcab_hostsim_eval(C.byref(obj), C.byref(prob), 1, sums.ctypes.data_as(C.c_void_p)) == 0
    t = torch.from_numpy(sums)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    rec = b.EvalRecord(); acc = np.zeros(m)
    assert sim.lib.sdcab_hostsim_eval_finish(C.byref(obj), C.c_int64(m), sums.ctypes.data_as(C.c_void_p),
                                             C.byref(rec), acc.ctypes.data_as(C.c_void_p)) == 0
    if kernel:
        whole = sim.evaluate(5, K, labels, A=A, kernel=True, c=1.0, gamma=0.5, k=1)
    else:
        whole = sim.evaluate(5, X, labels, A=A, W=W, c=1.0, gamma=0.5, k=1)
    got = b.record_to_dict(rec, acc)
    ok = all(abs(got[f] - whole[f]) <= 1e-12 * max(1, abs(whole[f])) for f in
             ("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer", "dual_regularizer"))
    ok = ok and np.allclose(got["accuracy"], whole["accuracy"], atol=1e-15)
    open(os.path.join(out_dir, "rank%d.txt" % rank), "w").write("ok" if ok else "mismatch %r %r" % (got, whole))
    dist.destroy_process_group()


@pytest.mark.parametrize("kernel", [False, True])
def test_two_rank_sums_equal_unsharded(tmp_path, kernel):
    import torch.multiprocessing as mp
    # A rank writes its result before it leaves the process group; a rendezvous that loses
    # the race for its port, or a worker that dies while the interpreter shuts down after
    # the result is on disk, is retried once with a new port.
    failure = None
    for attempt in range(2):
        out = tmp_path / ("attempt%d" % attempt)
        out.mkdir()
        try:
            mp.spawn(_worker, args=(2, _free_port(), kernel, str(out)), nprocs=2, join=True)
        except Exception as e:          # noqa: BLE001 - the result files decide
            failure = e
        results = [(out / ("rank%d.txt" % r)) for r in range(2)]
        if all(v.exists() for v in results):
            for v in results:
                assert v.read_text() == "ok"
            return
    raise AssertionError("no result from the ranks: %r" % (failure,))
