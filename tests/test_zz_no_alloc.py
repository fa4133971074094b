"""The evaluation entry point that allocates nothing.

Some hosts of this library are not allowed to allocate device memory while they
run (their own allocator owns the GPU, or they cannot afford the implicit
synchronisation of cudaMalloc).  For them the library carries a fixed scratch
array and ``sdcab_eval_sums_fixed_scratch_*_dev`` evaluates with it.  This test
calls that entry point through the C ABI twice in a row and checks both results
against the ordinary entry point and against the reference's evaluate_dataset;
the array is shared between calls, so the second call also proves that nothing
stale from the first one leaks in.  A further test reads the driver's count of
free device memory around the calls.
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


def test_fixed_scratch_matches_ordinary_entry_point(cuda_lib, ref):
    import torch
    from libsdca_b200 import binding as b
    lib = cuda_lib.lib()
    lib.sdcab_eval_fixed_scratch_bytes.restype = C.c_size_t
    lib.sdcab_eval_fixed_scratch_error.restype = C.c_char_p
    assert lib.sdcab_eval_fixed_scratch_bytes() == 16 << 20

    rng = np.random.default_rng(99)
    cases = [
        # objective id, reference's name, dtype, n, d, m, kernel
        (3, "l2_hinge_topk_smooth", np.float32, 9000, 48, 1000, False),   # several chunks through the 16 MiB array
        (5, "l2_topk_hinge_smooth", np.float64, 700, 20, 33, False),
        (1, "l2_entropy_topk", np.float64, 300, 300, 12, True),
    ]
    for oid, ref_name, dtype, n, d, m, kernel in cases:
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
        oracle = ref.evaluate(ref_name, X, A, labels, W=None if kernel else W, kernel=kernel,
                              c=1.0, gamma=0.5, k=2)
        tol = 1e-5 if dtype == np.float32 else 1e-12
        for attempt in range(2):   # two calls in a row share the array
            rc, got = sums_via(lib, "sdcab_eval_sums_fixed_scratch_%s_dev" % suffix, obj, prob, m)
            assert rc == 0, lib.sdcab_eval_fixed_scratch_error()
            assert lib.sdcab_eval_fixed_scratch_error() == b""
            assert np.all(np.abs(got[:8] - want[:8]) <= tol * np.maximum(1, np.abs(want[:8]))), (oid, attempt)
            # rank counts: equal, except that float32 scores from two GEMM kernels may
            # order a near-tie differently
            slack = 0 if dtype == np.float64 else max(4, n // 500)
            assert np.abs(got[8:] - want[8:]).sum() <= slack, (oid, attempt)
            # and against the reference's own evaluate_dataset, term by term (for float32
            # data the reference sums ||W||^2 in float: the regulariser terms, and the
            # totals that contain them, are compared with the exact double value instead)
            rec = b.eval_finish(obj, m, got)
            if dtype == np.float32:
                exact = 0.5 * float((W.astype(np.float64) ** 2).sum())
                assert abs(rec["primal_regularizer"] - exact) <= 1e-12 * exact
                fields = ("primal_loss", "dual_loss")
            else:
                fields = ("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer",
                          "dual_regularizer")
            for f in fields:
                assert abs(rec[f] - oracle[f]) <= tol * max(1, abs(oracle[f])), (oid, attempt, f)
            assert np.abs(rec["accuracy"] - oracle["accuracy"]).max() <= (2.0 / n if dtype == np.float32 else 1e-12)


def test_fixed_scratch_calls_allocate_nothing(cuda_lib):
    """Free device memory as the driver reports it does not move across calls of the
    entry point (after the first call on the device, which looks up the array's address
    and lets the runtime load the kernels)."""
    import torch
    from libsdca_b200 import binding as b
    lib = cuda_lib.lib()
    rng = np.random.default_rng(7)
    n, d, m = 6000, 64, 1000
    t = lambda a: torch.from_numpy(a).cuda()
    X = t(rng.standard_normal((n, d)).astype(np.float32))
    labels = t(rng.integers(0, m, n).astype(np.int64))
    A = t((-np.abs(rng.standard_normal((n, m))) * 0.01).astype(np.float32))
    W = t(rng.standard_normal((m, d)).astype(np.float32))
    sums = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    obj = b.make_objective(2, c=1.0, gamma=0.0, k=5)
    prob = b.make_problem(X, labels, A=A, W=W)
    call = lambda: lib.sdcab_eval_sums_fixed_scratch_f32_dev(C.byref(obj), C.byref(prob),
                                                            C.c_void_p(sums.data_ptr()), None)
    assert call() == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)


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


def test_fixed_scratch_rejects_rows_too_long_for_shared_memory(cuda_lib):
    """Between the two limits: 20 000 float classes fit the 16 MiB array but not the
    shared memory of the loss stage; the reason is readable."""
    import torch
    from libsdca_b200 import binding as b
    lib = cuda_lib.lib()
    lib.sdcab_eval_fixed_scratch_error.restype = C.c_char_p
    m, n, d = 20000, 4, 2
    X = torch.zeros((n, d), dtype=torch.float32, device="cuda")
    W = torch.zeros((m, d), dtype=torch.float32, device="cuda")
    A = torch.zeros((n, m), dtype=torch.float32, device="cuda")
    labels = torch.zeros(n, dtype=torch.int64, device="cuda")
    obj = b.make_objective(0, c=1.0)
    prob = b.make_problem(X, labels, A=A, W=W)
    sums = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    rc = lib.sdcab_eval_sums_fixed_scratch_f32_dev(C.byref(obj), C.byref(prob),
                                                   C.c_void_p(sums.data_ptr()), None)
    assert rc == -22
    assert b"shared memory" in lib.sdcab_eval_fixed_scratch_error()
