"""The evaluation entry point that allocates nothing.

Some hosts of this library are not allowed to allocate device memory while they
run (their own allocator owns the GPU, or they cannot afford the implicit
synchronisation of cudaMalloc).  For them the library carries a fixed scratch
array and ``sdcab_eval_sums_fixed_scratch_*_dev`` evaluates with it.  This test
calls that entry point through the C ABI twice in a row and checks both results
against the ordinary entry point; the array is shared between calls, so the
second call also proves that nothing stale from the first one leaks in.
Collected last on purpose: a failure here cannot hide the result of any other
test in a run that stops at the first failure.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def sums_via(lib, name, obj, prob, m, stream=None):
    import torch
    sums = torch.full((8 + m,), 123.0, dtype=torch.float64, device="cuda")  # stale on purpose
    fn = getattr(lib, name)
    if "fixed_scratch" in name:
        rc = fn(C.byref(obj), C.byref(prob), C.c_void_p(sums.data_ptr()), stream)
    else:
        rc = fn(C.byref(obj), C.byref(prob), C.c_void_p(sums.data_ptr()), None, C.c_size_t(0), stream)
    torch.cuda.synchronize()
    return rc, sums.cpu().numpy()


def test_fixed_scratch_matches_ordinary_entry_point(cuda_lib):
    import torch
    from libsdca_b200 import binding as b
    lib = cuda_lib.lib()
    lib.sdcab_eval_fixed_scratch_bytes.restype = C.c_size_t
    lib.sdcab_eval_fixed_scratch_error.restype = C.c_char_p
    assert lib.sdcab_eval_fixed_scratch_bytes() == 16 << 20

    rng = np.random.default_rng(99)
    cases = [
        # objective id, dtype, n, d, m, kernel
        (3, np.float32, 9000, 48, 1000, False),   # several chunks through the 16 MiB array
        (5, np.float64, 700, 20, 33, False),
        (1, np.float64, 300, 300, 12, True),
    ]
    for oid, dtype, n, d, m, kernel in cases:
        X = rng.standard_normal((n, d)).astype(dtype)
        labels = rng.integers(0, m, n).astype(np.int64)
        A = (-np.abs(rng.standard_normal((n, m))) * 0.01).astype(dtype)
        A[np.arange(n), labels] = 0.05
        W = rng.standard_normal((m, d)).astype(dtype)
        t = lambda a: torch.from_numpy(a).cuda()
        tX, tl, tA, tW = t(X), t(labels), t(A), t(W)
        obj = b.make_objective(oid, c=1.0, gamma=0.5, k=2)
        prob = b.make_problem(tX, tl, A=tA, W=None if kernel else tW, kernel=kernel)
        suffix = "f32" if dtype == np.float32 else "f64"
        rc, want = sums_via(lib, "sdcab_eval_sums_%s_dev" % suffix, obj, prob, m)
        assert rc == 0
        for attempt in range(2):   # two calls in a row share the array
            rc, got = sums_via(lib, "sdcab_eval_sums_fixed_scratch_%s_dev" % suffix, obj, prob, m)
            assert rc == 0, lib.sdcab_eval_fixed_scratch_error()
            tol = 1e-5 if dtype == np.float32 else 1e-12
            assert np.all(np.abs(got[:8] - want[:8]) <= tol * np.maximum(1, np.abs(want[:8]))), (oid, attempt)
            # rank counts: equal, except that float32 scores from the two GEMM kernels may
            # order a near-tie differently
            slack = 0 if dtype == np.float64 else max(4, n // 500)
            assert np.abs(got[8:] - want[8:]).sum() <= slack, (oid, attempt)


def test_fixed_scratch_rejects_what_does_not_fit(cuda_lib):
    import torch
    from libsdca_b200 import binding as b
    lib = cuda_lib.lib()
    lib.sdcab_eval_fixed_scratch_error.restype = C.c_char_p
    m, n, d = 70000, 4, 2   # 32 rows of 70 000 doubles exceed 16 MiB
    X = torch.zeros((n, d), dtype=torch.float64, device="cuda")
    W = torch.zeros((m, d), dtype=torch.float64, device="cuda")
    A = torch.zeros((n, m), dtype=torch.float64, device="cuda")
    labels = torch.zeros(n, dtype=torch.int64, device="cuda")
    obj = b.make_objective(0, c=1.0)
    prob = b.make_problem(X, labels, A=A, W=W)
    sums = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    rc = lib.sdcab_eval_sums_fixed_scratch_f64_dev(C.byref(obj), C.byref(prob),
                                                   C.c_void_p(sums.data_ptr()), None)
    assert rc == -22
    assert b"fixed scratch" in lib.sdcab_eval_fixed_scratch_error()
