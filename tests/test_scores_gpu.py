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
          (513, 100, 129), (128, 16, 128), (257, 4096, 1000), (129, 33, 5), (64, 32, 128)]


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
