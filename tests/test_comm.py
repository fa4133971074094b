"""The communicator of the sharded gap evaluation (NCCL behind the C ABI)."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from libsdca_b200 import binding as b

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_argument_handling_needs_no_gpu():
    lib = b.lib()
    # no communicator = one shard: the reductions are no-ops, rank / size are defined
    assert lib.sdcab_comm_allreduce_f64(None, None, C.c_int64(0), None) == 0
    assert lib.sdcab_comm_rank(None) == -1 and lib.sdcab_comm_size(None) == 0
    assert lib.sdcab_comm_destroy(None) == 0
    h = C.c_void_p()
    ident = C.create_string_buffer(128)
    assert lib.sdcab_comm_create(C.byref(h), 0, 0, ident) == -1         # nranks < 1
    assert lib.sdcab_comm_create(C.byref(h), 2, 2, ident) == -1         # rank out of range
    assert lib.sdcab_comm_create(None, 1, 0, ident) == -1
    assert lib.sdcab_comm_unique_id(None) == -1
    assert lib.sdcab_status_string(-24) == b"nccl_error"


@pytest.mark.gpu
def test_one_rank_communicator_is_the_plain_evaluation(cuda_lib):
    import torch
    rng = np.random.default_rng(2)
    n, d, m = 500, 64, 20
    t = lambda a: torch.from_numpy(a).cuda()
    X = t(rng.standard_normal((n, d)).astype(np.float32))
    labels = t(rng.integers(0, m, n).astype(np.int64))
    A = t((-np.abs(rng.standard_normal((n, m))) * 0.01).astype(np.float32))
    W = t(rng.standard_normal((m, d)).astype(np.float32))
    obj = b.make_objective("topk_hinge_alpha", c=1.0, gamma=0.0, k=3)
    prob = b.make_problem(X, labels, A=A, W=W)
    plain = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    cuda_lib.eval_sums_(obj, prob, plain, "f32")
    comm = b.Comm.create(1, 0, b.Comm.unique_id())
    try:
        assert cuda_lib.lib().sdcab_comm_size(comm.handle) == 1
        sharded = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
        comm.eval_sums_(obj, prob, sharded, "f32")
        torch.cuda.synchronize()
        assert torch.equal(plain, sharded)
        v = torch.arange(5, dtype=torch.float32, device="cuda")
        assert torch.equal(comm.allreduce_(v.clone()), v)
    finally:
        comm.destroy()


WORKER = r"""
import os, sys
sys.path.insert(0, %r)
import numpy as np, torch
import libsdca_b200 as sd
from libsdca_b200 import binding as b
rank, world, path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
torch.cuda.set_device(rank)
if rank == 0:
    open(path + ".tmp", "wb").write(b.Comm.unique_id()); os.replace(path + ".tmp", path)
import time
for _ in range(600):
    if os.path.exists(path): break
    time.sleep(0.05)
ident = open(path, "rb").read()
comm = b.Comm.create(world, rank, ident)
rng = np.random.default_rng(7)
n, d, m = 900, 48, 12
X = rng.standard_normal((n, d)); labels = rng.integers(0, m, n).astype(np.int64)
A = -np.abs(rng.standard_normal((n, m))) * 0.01; A[np.arange(n), labels] = 0.04
W = rng.standard_normal((m, d))
lo, hi = (n * rank) // world, (n * (rank + 1)) // world
t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
obj = b.make_objective("l2_entropy_topk", c=1.0, k=2)
prob = b.make_problem(t(X[lo:hi]), t(labels[lo:hi]), A=t(A), W=t(W), a_row_offset=lo,
                      include_primal_regularizer=(rank == 0))
sums = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
comm.eval_sums_(obj, prob, sums, "f64")
torch.cuda.synchronize()
np.save(path + ".rank%%d.npy" %% rank, sums.cpu().numpy())
comm.destroy()
""" % ROOT


@pytest.mark.gpu
def test_two_ranks_add_their_shards(cuda_lib, ref, tmp_path):
    """Two processes, one GPU each: the all-reduced sums of the two shards are the sums of
    the whole set on both ranks, and finish to the reference's record."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    path = str(tmp_path / "nccl_id")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", WORKER, str(r), "2", path], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err[-2000:]
    s0, s1 = (np.load(path + ".rank%d.npy" % r) for r in range(2))
    assert np.array_equal(s0, s1)
    rng = np.random.default_rng(7)
    n, d, m = 900, 48, 12
    X = rng.standard_normal((n, d)); labels = rng.integers(0, m, n).astype(np.int64)
    A = -np.abs(rng.standard_normal((n, m))) * 0.01; A[np.arange(n), labels] = 0.04
    W = rng.standard_normal((m, d))
    rec = b.eval_finish(b.make_objective("l2_entropy_topk", c=1.0, k=2), m, s0)
    r = ref.evaluate("l2_entropy_topk", X, A, labels, W=W, c=1.0, k=2)
    for f in ("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer", "dual_regularizer"):
        assert abs(rec[f] - r[f]) <= 1e-12 * max(1, abs(r[f])), f
    assert np.abs(rec["accuracy"] - r["accuracy"]).max() <= 1e-12
