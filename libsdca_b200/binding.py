"""ctypes binding of ``libsdca_b200.so``.

The calling conventions mirror the reference's Matlab front end: ``prox`` takes
the matrix whose rows are the vectors (the same memory as Matlab's m x N
column-major array) and an option set with the defaults of ``matsdca_prox``
(src/matlab/mex_prox.cpp:121-127 of the reference).

numpy arrays go through the host-buffer entry points (the library copies to the
device and back); torch CUDA tensors go through the ``*_dev`` entry points on
the current torch stream, in place.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

PROX_NAMES = (
    "knapsack", "knapsack_eq", "knapsack_le", "knapsack_le_biased", "topk_simplex",
    "topk_simplex_biased", "topk_cone", "topk_cone_biased", "entropy", "entropy_norm",
    "topk_entropy", "topk_entropy_biased", "two_simplex", "two_simplex_sort",
    "lambert_w_exp",
)


class SdcabError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        msg = "%s failed: %s (%d)" % (where, status_string(status), status)
        detail = lib().sdcab_last_error().decode()
        if detail:
            msg += " -- " + detail
        super().__init__(msg)


class ProxOpts(C.Structure):
    _fields_ = [("lo", C.c_double), ("hi", C.c_double), ("rhs", C.c_double),
                ("rho", C.c_double), ("alpha", C.c_double), ("k", C.c_int64),
                ("p", C.c_int64), ("precision", C.c_int32), ("reserved", C.c_int32)]


class Thresholds(C.Structure):
    _fields_ = [("t", C.c_double), ("lo", C.c_double), ("hi", C.c_double),
                ("num_hi", C.c_int32), ("num_mid", C.c_int32)]


THR_DTYPE = np.dtype([("t", "<f8"), ("lo", "<f8"), ("hi", "<f8"),
                      ("num_hi", "<i4"), ("num_mid", "<i4")])

_lib = None


def library_path():
    return os.path.join(HERE, "libsdca_b200.so")


def lib():
    """The loaded shared library; building it is ``python -m libsdca_b200.build``."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise ImportError(
                "%s is missing: build it with `python -m libsdca_b200.build` "
                "(there is no CPU fallback)" % path)
        _lib = C.CDLL(path)
        _lib.sdcab_status_string.restype = C.c_char_p
        _lib.sdcab_last_error.restype = C.c_char_p
        _lib.sdcab_version.restype = C.c_char_p
    return _lib


def status_string(status):
    return lib().sdcab_status_string(int(status)).decode()


def _check(rc, where):
    if rc != 0:
        raise SdcabError(rc, where)


def make_opts(lo=0.0, hi=1.0, rhs=1.0, rho=1.0, alpha=1.0, k=1, p=1, precision="double"):
    prec = {"double": 0, "single": 1, "float": 1}.get(precision)
    if prec is None:
        # "long double" exists in the reference's front end but has no device type
        raise SdcabError(-8, "precision=%r" % (precision,))
    return ProxOpts(lo, hi, rhs, rho, alpha, int(k), int(p), prec, 0)


def _is_torch(x):
    return type(x).__module__.startswith("torch")


def _suffix(dtype_name):
    if dtype_name in ("float32", "torch.float32"):
        return "f32"
    if dtype_name in ("float64", "torch.float64"):
        return "f64"
    raise SdcabError(-3, "dtype %s" % dtype_name)


def _torch_stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def prox_(a, prox="knapsack", **opts):
    """In-place batched prox on the rows of ``a`` (numpy C-contiguous or torch CUDA)."""
    o = make_opts(**opts)
    if _is_torch(a):
        if not (a.is_cuda and a.is_contiguous() and a.dim() == 2):
            raise SdcabError(-1, "prox_: contiguous 2-d CUDA tensor expected")
        n, m = a.shape
        fn = getattr(lib(), "sdcab_prox_%s_dev" % _suffix(str(a.dtype)))
        _check(fn(prox.encode(), C.c_void_p(a.data_ptr()), C.c_int64(m), C.c_int64(n),
                  C.byref(o), _torch_stream()), "sdcab_prox_dev(%s)" % prox)
        return a
    if not (isinstance(a, np.ndarray) and a.ndim == 2 and a.flags.c_contiguous):
        raise SdcabError(-1, "prox_: C-contiguous 2-d array expected")
    n, m = a.shape
    fn = getattr(lib(), "sdcab_prox_%s" % _suffix(a.dtype.name))
    _check(fn(prox.encode(), a.ctypes.data_as(C.c_void_p), C.c_int64(m), C.c_int64(n),
              C.byref(o), None), "sdcab_prox(%s)" % prox)
    return a


def prox_to(a, out, prox="knapsack", **opts):
    """Device form with separate input and output tensors (torch CUDA, same shape)."""
    o = make_opts(**opts)
    n, m = a.shape
    fn = getattr(lib(), "sdcab_prox_to_%s_dev" % _suffix(str(a.dtype)))
    _check(fn(prox.encode(), C.c_void_p(a.data_ptr()), C.c_void_p(out.data_ptr()),
              C.c_int64(m), C.c_int64(n), C.byref(o), _torch_stream()),
           "sdcab_prox_to_dev(%s)" % prox)
    return out


def prox(a, prox="knapsack", **opts):
    """Like ``matsdca_prox(A, opts)`` with an output argument: returns a new matrix."""
    if _is_torch(a):
        return prox_(a.clone(), prox, **opts)
    return prox_(np.array(a, order="C", copy=True), prox, **opts)


def thresholds(a, prox="knapsack", **opts):
    """Per-row (t, lo, hi, num_hi, num_mid) as a numpy structured array."""
    o = make_opts(**opts)
    two = prox in ("two_simplex", "two_simplex_sort")
    if _is_torch(a):
        import torch
        n, m = a.shape
        cnt = 2 * n if two else n
        out = torch.empty(cnt * THR_DTYPE.itemsize, dtype=torch.uint8, device=a.device)
        fn = getattr(lib(), "sdcab_thresholds_%s_dev" % _suffix(str(a.dtype)))
        _check(fn(prox.encode(), C.c_void_p(a.data_ptr()), C.c_int64(m), C.c_int64(n),
                  C.byref(o), C.c_void_p(out.data_ptr()), _torch_stream()),
               "sdcab_thresholds_dev(%s)" % prox)
        return out.cpu().numpy().view(THR_DTYPE)
    a = np.ascontiguousarray(a)
    n, m = a.shape
    out = np.zeros(2 * n if two else n, dtype=THR_DTYPE)
    fn = getattr(lib(), "sdcab_thresholds_%s" % _suffix(a.dtype.name))
    _check(fn(prox.encode(), a.ctypes.data_as(C.c_void_p), C.c_int64(m), C.c_int64(n),
              C.byref(o), out.ctypes.data_as(C.c_void_p)), "sdcab_thresholds(%s)" % prox)
    return out


def lambert_w_exp_(x):
    """x <- W(exp(x)) elementwise, in place (torch CUDA tensor or numpy array)."""
    if _is_torch(x):
        fn = getattr(lib(), "sdcab_lambert_w_exp_%s_dev" % _suffix(str(x.dtype)))
        _check(fn(C.c_void_p(x.data_ptr()), C.c_int64(x.numel()), _torch_stream()),
               "sdcab_lambert_w_exp_dev")
        return x
    flat = x.reshape(1, -1)
    prox_(flat, "lambert_w_exp")
    return x
