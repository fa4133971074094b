"""The shared library loads without a GPU and exports every symbol that
include/sdca_b200.h declares; argument errors are reported as status codes."""
import ctypes as C
import os
import re
import shutil

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import libsdca_b200
    if not os.path.exists(libsdca_b200.library_path()):
        if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
            pytest.skip("library not built and nvcc unavailable")
        from libsdca_b200 import build
        build.build()
    return libsdca_b200.lib()


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        text = open(os.path.join(inc, f)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(sdcab_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_exports_every_declared_symbol(lib):
    names = declared_symbols()
    assert len(names) >= 10
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_status_strings(lib):
    assert lib.sdcab_status_string(0) == b"ok"
    assert lib.sdcab_status_string(-6) == b"LIBSDCA:prox"
    assert lib.sdcab_status_string(-8) == b"LIBSDCA:precision"


def test_argument_errors_need_no_gpu(lib):
    from libsdca_b200.binding import ProxOpts
    o = ProxOpts()
    lib.sdcab_prox_opts_default(C.byref(o))
    assert (o.lo, o.hi, o.rhs, o.rho, o.alpha, o.k, o.p) == (0, 1, 1, 1, 1, 1, 1)
    buf = (C.c_float * 8)()
    f = lib.sdcab_prox_f32_dev
    assert f(b"no_such_prox", buf, C.c_int64(4), C.c_int64(2), C.byref(o), None) == -6
    assert f(b"topk_simplex", buf, C.c_int64(0), C.c_int64(2), C.byref(o), None) == -4
    o.k = 9
    assert f(b"topk_simplex", buf, C.c_int64(4), C.c_int64(2), C.byref(o), None) == -2
    o.k = 1; o.alpha = 0.0
    assert f(b"topk_entropy_biased", buf, C.c_int64(4), C.c_int64(2), C.byref(o), None) == -2
    o.alpha = 1.0; o.precision = 7
    assert f(b"knapsack", buf, C.c_int64(4), C.c_int64(2), C.byref(o), None) == -8


def test_epoch_order_needs_no_gpu(lib):
    """sdcab_epoch_permutations is host code: the committed orders of the reference's
    solver (std::minstd_rand + std::shuffle) come out of the product library."""
    import numpy as np
    from tests.golden_util import epoch_orders
    big, small = epoch_orders()
    perm = np.zeros((3, 1000), dtype=np.int64)
    assert lib.sdcab_epoch_permutations(C.c_int64(1000), C.c_int64(3), perm.ctypes.data_as(C.c_void_p)) == 0
    assert np.array_equal(perm, small)
    perm = np.zeros((2, 50000), dtype=np.int64)
    assert lib.sdcab_epoch_permutations(C.c_int64(50000), C.c_int64(2), perm.ctypes.data_as(C.c_void_p)) == 0
    assert np.array_equal(perm[:, :64], big)
    assert lib.sdcab_epoch_permutations(C.c_int64(-1), C.c_int64(1), None) != 0
