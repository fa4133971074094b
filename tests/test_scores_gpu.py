"""The score GEMMs (tensor-core 3xTF32 for float features, CUDA-core FMA
otherwise) against a float64 product, through sdcab_scores_*_dev."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SHAPES = [(300, 64, 1000), (130, 12, 7), (70, 37, 133), (300, 64, 1024), (1, 4096, 1000),
          (513, 100, 129), (128, 16, 128), (257, 4096, 1000), (129, 33, 5), (64, 32, 128),
          # the paired tensor-core kernel is persistent: more 256 x 256 tiles than SM pairs
          # (several tiles per pair, accumulators handed over across tile boundaries), a
          # contraction shorter than one accumulation chunk, ragged last tiles
          (5000, 64, 1000), (9000, 1024, 1000), (700, 96, 300), (256, 32, 256), (255, 36, 257)]


def scores(mod, X, W=None, A=None):
    import torch
    from libsdca_b200 import binding as b
    n = X.shape[0]
    m = W.shape[0] if W is not None else A.shape[1]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    tX, tl = t(X), t(np.zeros(n, dtype=np.int64))
    if W is not None:
        keep = t(W)
        p = b.make_problem(tX, tl, W=keep, is_train=False)
    else:
        keep = t(A)
        p = b.make_problem(tX, tl, A=keep, kernel=True, is_train=False)
    out = torch.zeros((n, m), dtype=tX.dtype, device="cuda")
    fn = getattr(mod.lib(), "sdcab_scores_%s_dev" % ("f32" if X.dtype == np.float32 else "f64"))
    rc = fn(C.byref(p), C.c_void_p(out.data_ptr()), None)
    torch.cuda.synchronize()
    assert rc == 0, rc
    return out.cpu().numpy()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_scores_match_float64_product(cuda_lib, dtype):
    rng = np.random.default_rng(0)
    for n, d, m in SHAPES:
        X = rng.standard_normal((n, d)).astype(dtype)
        W = rng.standard_normal((m, d)).astype(dtype)
        A = rng.standard_normal((d, m)).astype(dtype)
        # error of a length-d dot product in the data type, relative to sum |x||w|:
        # a few ulps plus the usual sqrt(d) growth
        eps = np.finfo(dtype).eps
        for got, ref, mag in ((scores(cuda_lib, X, W=W), X.astype(np.float64) @ W.astype(np.float64).T,
                               np.abs(X).astype(np.float64) @ np.abs(W).astype(np.float64).T),
                              (scores(cuda_lib, X, A=A), X.astype(np.float64) @ A.astype(np.float64),
                               np.abs(X).astype(np.float64) @ np.abs(A).astype(np.float64))):
            bound = (16 + 2 * np.sqrt(d)) * eps * mag
            assert (np.abs(got - ref) <= bound + 1e-30).all(), (n, d, m, np.abs(got - ref).max())


def test_tensor_core_and_cuda_core_gemm_agree(cuda_lib):
    """The library's test switch forces the CUDA-core kernel: both must agree to float
    accuracy, and they are two different kernels."""
    from libsdca_b200 import binding as b
    rng = np.random.default_rng(3)
    X = rng.standard_normal((384, 1024)).astype(np.float32)
    W = rng.standard_normal((1000, 1024)).astype(np.float32)
    outs = []
    try:
        for simt in (0, 1):
            b.test_set("gemm_simt", simt)
            outs.append(scores(cuda_lib, X, W=W))
    finally:
        b.test_set("gemm_simt", 0)
    assert not np.array_equal(outs[0], outs[1])          # two different kernels really ran
    assert np.abs(outs[0] - outs[1]).max() <= 1e-5 * np.abs(outs[1]).max()


def test_double_precision_tiles_agree(cuda_lib):
    """The three tiles of the double-precision product (the 128-column block tile, the
    pipelined 104-column tile with 64 and with 128 rows per block) on shapes with ragged
    edges in every direction, odd leading dimensions (8-byte copies) and both operand
    forms: each within the dot-product bound of the exact result, and the forced tiles
    really are different kernels from one another where the shape lets them differ."""
    from libsdca_b200 import binding as b
    rng = np.random.default_rng(17)
    shapes = [(333, 50, 100), (130, 17, 7), (64, 16, 104), (700, 129, 105), (257, 1000, 99),
              (19000, 40, 100), (45, 3, 3)]
    eps = np.finfo(np.float64).eps
    try:
        for n, d, m in shapes:
            X = rng.standard_normal((n, d))
            W = rng.standard_normal((m, d))
            A = rng.standard_normal((d, m))
            for kw, exact, mag in ((dict(W=W), X @ W.T, np.abs(X) @ np.abs(W).T),
                                   (dict(A=A), X @ A, np.abs(X) @ np.abs(A))):
                outs = []
                for mode in (1, 2, 3, 0):
                    b.test_set("gemm_f64_tile", mode)
                    outs.append(scores(cuda_lib, X, **kw))
                    assert (np.abs(outs[-1] - exact) <= (16 + 2 * np.sqrt(d)) * eps * mag + 1e-300).all(), \
                        (n, d, m, mode)
                # the two pipelined tiles add the same terms in the same order
                assert np.array_equal(outs[1], outs[2]), (n, d, m)
    finally:
        b.test_set("gemm_f64_tile", 0)


def test_tensor_core_variants_agree(cuda_lib):
    """The paired-CTA kernel leaves the truncation of an operand to TF32 to the tensor
    core; with the head written explicitly (test switch) the result must be the same bit
    for bit, which is what shows that the hardware truncates.  The one-CTA kernel agrees
    to float accuracy (its sums run in a different order)."""
    from libsdca_b200 import binding as b
    rng = np.random.default_rng(13)
    X = rng.standard_normal((1000, 2048)).astype(np.float32)
    W = rng.standard_normal((600, 2048)).astype(np.float32)
    exact = X.astype(np.float64) @ W.astype(np.float64).T
    try:
        base = scores(cuda_lib, X, W=W)
        b.test_set("gemm_write_hi", 1)
        explicit = scores(cuda_lib, X, W=W)
        b.test_set("gemm_write_hi", 0)
        b.test_set("gemm_single_cta", 1)
        single = scores(cuda_lib, X, W=W)
    finally:
        b.test_set("gemm_write_hi", 0)
        b.test_set("gemm_single_cta", 0)
    assert np.array_equal(base, explicit)
    assert np.abs(base - single).max() <= 1e-5 * np.abs(single).max()
    mag = np.abs(X).astype(np.float64) @ np.abs(W).astype(np.float64).T
    eps = np.finfo(np.float32).eps
    for got in (base, single):
        assert (np.abs(got - exact) <= (16 + 2 * np.sqrt(2048)) * eps * mag).all()


def test_a_wait_that_runs_out_becomes_a_status(cuda_lib):
    """Every wait inside the tensor-core kernel is bounded.  With the test switch the
    kernel skips one operand tile and runs with a short limit, so that a wait really runs
    out: the roles leave their loops, tensor memory is freed, the call reports
    SDCAB_ERR_TIMEOUT, and the next call on the same context works."""
    import torch
    from libsdca_b200 import binding as b
    rng = np.random.default_rng(5)
    X = rng.standard_normal((512, 256)).astype(np.float32)
    W = rng.standard_normal((256, 256)).astype(np.float32)
    tX, tW = torch.from_numpy(X).cuda(), torch.from_numpy(W).cuda()
    labels = torch.zeros(512, dtype=torch.int64, device="cuda")
    p = b.make_problem(tX, labels, W=tW, is_train=False)
    out = torch.zeros((512, 256), dtype=torch.float32, device="cuda")
    fn = cuda_lib.lib().sdcab_scores_f32_dev
    try:
        b.test_set("gemm_lose_a_tile", 1)
        rc = fn(C.byref(p), C.c_void_p(out.data_ptr()), None)
    finally:
        b.test_set("gemm_lose_a_tile", 0)
    torch.cuda.synchronize()
    assert rc == -23, rc
    assert cuda_lib.lib().sdcab_status_string(rc) == b"device_wait_timeout"
    # the evaluation reports it through the sums vector's error word
    A = torch.zeros((512, 256), dtype=torch.float32, device="cuda")
    try:
        b.test_set("gemm_lose_a_tile", 1)
        with pytest.raises(cuda_lib.SdcabError) as e:
            cuda_lib.evaluate("msvm", tX, labels, A=A, W=tW)
        assert e.value.status == -23
    finally:
        b.test_set("gemm_lose_a_tile", 0)
    good = scores(cuda_lib, X, W=W)
    exact = X.astype(np.float64) @ W.astype(np.float64).T
    mag = np.abs(X).astype(np.float64) @ np.abs(W).astype(np.float64).T
    assert (np.abs(good - exact) <= (16 + 2 * np.sqrt(256)) * np.finfo(np.float32).eps * mag).all()
