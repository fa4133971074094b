"""numpy front end of the CPU checkers (test infrastructure, never a product path).

Two back ends share one calling convention:

* ``Reference``  -- ``oracle/_ref/libsdca_ref.so``: the reference's own headers,
  compiled unmodified by ``oracle/build_oracle.py``.
* ``Restatement`` -- ``oracle/libsdca_oracle.so``: the plain-C restatement of the
  same algorithms in ``oracle/sdca_oracle.c``.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

OBJECTIVES = {
    "l2_entropy": 0, "softmax": 0,
    "l2_entropy_topk": 1, "topk_softmax": 1,
    "l2_hinge_topk": 2, "topk_hinge_alpha": 2,
    "l2_hinge_topk_smooth": 3, "topk_hinge_alpha_smooth": 3,
    "l2_topk_hinge": 4, "topk_hinge_beta": 4, "msvm": 4,
    "l2_topk_hinge_smooth": 5, "topk_hinge_beta_smooth": 5, "msvm_smooth": 5,
    "l2_multilabel_hinge": 6, "mlsvm": 6,
    "l2_multilabel_hinge_smooth": 7, "mlsvm_smooth": 7,
    "l2_multilabel_entropy": 8, "mlsoftmax": 8,
}
MULTILABEL = {6, 7, 8}
EVAL_FIELDS = ("primal", "dual", "primal_loss", "dual_loss",
               "primal_regularizer", "dual_regularizer", "rank_loss")


class ProxOpts(C.Structure):
    _fields_ = [("lo", C.c_double), ("hi", C.c_double), ("rhs", C.c_double),
                ("rho", C.c_double), ("alpha", C.c_double),
                ("k", C.c_int64), ("p", C.c_int64)]


def make_opts(lo=0.0, hi=1.0, rhs=1.0, rho=1.0, alpha=1.0, k=1, p=1):
    return ProxOpts(lo, hi, rhs, rho, alpha, k, p)


class EvalArgs(C.Structure):
    _fields_ = [("objective", C.c_int), ("c", C.c_double), ("gamma", C.c_double),
                ("k", C.c_int64), ("input_kind", C.c_int), ("d", C.c_int64),
                ("n", C.c_int64), ("m", C.c_int64), ("X", C.c_void_p),
                ("A", C.c_void_p), ("W", C.c_void_p), ("W0", C.c_void_p),
                ("labels", C.c_void_p), ("offsets", C.c_void_p),
                ("is_train", C.c_int), ("nthreads", C.c_int),
                ("epsilon", C.c_double), ("max_epoch", C.c_int64),
                ("eval_epoch", C.c_int64), ("eval_on_start", C.c_int)]


class RefTestSet(C.Structure):
    _fields_ = [("n", C.c_int64), ("X", C.c_void_p), ("labels", C.c_void_p), ("offsets", C.c_void_p),
                ("out", C.c_void_p), ("acc", C.c_void_p)]


def _dtype_code(dt):
    dt = np.dtype(dt)
    if dt == np.float32:
        return 0
    if dt == np.float64:
        return 1
    raise TypeError("float32 or float64 expected")


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class _Backend:
    """Shared wrappers; ``prefix`` selects the exported symbol family."""

    prefix = None
    path = None

    def __init__(self):
        if not os.path.exists(self.path):
            raise FileNotFoundError(self.path)
        self.lib = C.CDLL(self.path)

    def _fn(self, name):
        return getattr(self.lib, self.prefix + name)

    def has(self, name):
        return hasattr(self.lib, self.prefix + name)

    # rows of ``a`` are the vectors (n x m, C order)
    def prox(self, name, a, result="double", nthreads=1, inplace=False, **kw):
        """``inplace=True`` works on ``a`` itself (C-contiguous), as matsdca_prox does when
        it is called without an output argument (src/matlab/mex_prox.cpp:113-119)."""
        if inplace:
            if not (isinstance(a, np.ndarray) and a.flags.c_contiguous and a.flags.writeable):
                raise ValueError("inplace needs a writeable C-contiguous array")
        else:
            a = np.array(a, order="C", copy=True)
        n, m = a.shape
        o = make_opts(**kw)
        rc = self._fn("prox")(name.encode(), _dtype_code(a.dtype),
                              _dtype_code(np.float64 if result == "double" else np.float32),
                              _ptr(a), C.c_int64(m), C.c_int64(n), C.byref(o), int(nthreads))
        if rc != 0:
            raise RuntimeError("%sprox(%s) -> %d" % (self.prefix, name, rc))
        return a

    def thresholds(self, name, a, result="double", **kw):
        a = np.ascontiguousarray(a)
        n, m = a.shape
        two = name in ("two_simplex", "two_simplex_sort")
        cnt = 2 * n if two else n
        t = np.zeros(cnt); lo = np.zeros(cnt); hi = np.zeros(cnt)
        nu = np.zeros(cnt, dtype=np.int64); nm = np.zeros(cnt, dtype=np.int64)
        o = make_opts(**kw)
        rc = self._fn("thresholds")(name.encode(), _dtype_code(a.dtype),
                                    _dtype_code(np.float64 if result == "double" else np.float32),
                                    _ptr(a), C.c_int64(m), C.c_int64(n), C.byref(o),
                                    _ptr(t), _ptr(lo), _ptr(hi), _ptr(nu), _ptr(nm))
        if rc != 0:
            raise RuntimeError("%sthresholds(%s) -> %d" % (self.prefix, name, rc))
        return dict(t=t, lo=lo, hi=hi, num_hi=nu, num_mid=nm)

    def _eval_args(self, objective, X, A, labels, W=None, W0=None, offsets=None,
                   kernel=False, c=1.0, gamma=0.0, k=1, is_train=True, nthreads=1):
        obj = OBJECTIVES[objective] if isinstance(objective, str) else int(objective)
        # X: (n, d) C order == d x n column major; kernel: (n, n_train) C order.
        n, d = X.shape
        m = A.shape[1] if A is not None else W.shape[0]
        a = EvalArgs()
        a.objective = obj; a.c = c; a.gamma = gamma; a.k = k
        a.input_kind = 1 if kernel else 0
        a.d = d; a.n = n; a.m = m
        a.X = X.ctypes.data; a.A = A.ctypes.data if A is not None else None
        a.W = W.ctypes.data if W is not None else None
        a.W0 = W0.ctypes.data if W0 is not None else None
        a.labels = labels.ctypes.data
        a.offsets = offsets.ctypes.data if offsets is not None else None
        a.is_train = 1 if is_train else 0
        a.nthreads = nthreads
        return a, m

    def evaluate(self, objective, X, A, labels, result="double", **kw):
        """X: (n, d) features or (n, n_train) kernel rows; A: (n_train, m); W: (m, d)."""
        a, m = self._eval_args(objective, X, A, labels, **kw)
        out = np.zeros(8); acc = np.zeros(m)
        rc = self._fn("eval")(C.byref(a), _dtype_code(X.dtype),
                              _dtype_code(np.float64 if result == "double" else np.float32),
                              _ptr(out), _ptr(acc))
        if rc != 0:
            raise RuntimeError("%seval -> %d" % (self.prefix, rc))
        rec = {f: out[i] for i, f in enumerate(EVAL_FIELDS)}
        rec["accuracy"] = acc
        return rec

    def fit(self, objective, X, A, labels, epsilon=1e-3, max_epoch=1000, eval_epoch=10,
            eval_on_start=False, result="double", tests=None, **kw):
        """``tests``: held-out sets as (X, labels[, offsets]) tuples (reference back end only);
        the result then has ``tests``: per set a dict of primal_loss, rank_loss (one entry per
        evaluation) and accuracy (evaluations x m)."""
        a, m = self._eval_args(objective, X, A, labels, **kw)
        test_out = []
        if tests:
            cap_t = max_epoch + 4
            sets = (RefTestSet * len(tests))()
            for i, t in enumerate(tests):
                out = np.zeros((cap_t, 2)); acc = np.zeros((cap_t, m))
                sets[i].n = t[0].shape[0]; sets[i].X = t[0].ctypes.data; sets[i].labels = t[1].ctypes.data
                sets[i].offsets = t[2].ctypes.data if len(t) > 2 and t[2] is not None else None
                sets[i].out = out.ctypes.data; sets[i].acc = acc.ctypes.data
                test_out.append((out, acc))
            self._fn("set_tests")(sets, len(tests), C.c_int64(cap_t))
        a.epsilon = epsilon; a.max_epoch = max_epoch; a.eval_epoch = eval_epoch
        a.eval_on_start = 1 if eval_on_start else 0
        cap = max_epoch + 4
        hist = np.zeros((cap, 8)); acc = np.zeros(m)
        ne = C.c_int64(0); ep = C.c_int64(0); st = C.c_int(0)
        rc = self._fn("fit")(C.byref(a), _dtype_code(X.dtype),
                             _dtype_code(np.float64 if result == "double" else np.float32),
                             _ptr(hist), C.c_int64(cap), C.byref(ne), C.byref(ep),
                             C.byref(st), _ptr(acc))
        if rc != 0:
            raise RuntimeError("%sfit -> %d" % (self.prefix, rc))
        res = dict(history=hist[:ne.value].copy(), epoch=ep.value, status=st.value, accuracy=acc)
        if tests:
            res["tests"] = [dict(primal_loss=o[:ne.value, 0].copy(), rank_loss=o[:ne.value, 1].copy(),
                                 accuracy=ac[:ne.value].copy()) for o, ac in test_out]
        return res

    def epoch_permutations(self, n, num_epochs):
        perm = np.zeros((num_epochs, n), dtype=np.int64)
        self._fn("epoch_permutations")(C.c_int64(n), C.c_int64(num_epochs), _ptr(perm))
        return perm

    def lambert_w_exp(self, x):
        x = np.asarray(x)
        if x.dtype == np.float32:
            f = self._fn("lambert_w_exp_f32"); f.restype = C.c_float; f.argtypes = [C.c_float]
        else:
            f = self._fn("lambert_w_exp_f64"); f.restype = C.c_double; f.argtypes = [C.c_double]
        return np.array([f(v) for v in x.ravel().tolist()], dtype=x.dtype).reshape(x.shape)


class Reference(_Backend):
    prefix = "sdca_ref_"
    path = os.path.join(HERE, "_ref", "libsdca_ref.so")

    def use_blas(self, path, num_threads=1):
        return self.lib.sdca_ref_use_blas(path.encode() if path else None, int(num_threads))


class ReferenceAccurate(Reference):
    """The same headers compiled with SDCA_ACCURATE_MATH."""
    path = os.path.join(HERE, "_ref", "libsdca_ref_accurate.so")


class Restatement(_Backend):
    prefix = "sdca_oracle_"
    path = os.path.join(HERE, "libsdca_oracle.so")

    def two_simplex_sort_defined(self, a, p=1, rhs=1.0, result="double", **_):
        """Rows on which the reference's two_simplex_sort stays inside its arrays
        (prox/two_simplex_sort.h:84-97): worked out by the restatement's memory-safe walk,
        never by running the reference on a row that would read past a block."""
        a = np.ascontiguousarray(a)
        n, m = a.shape
        flags = np.zeros(n, dtype=np.int32)
        rc = self._fn("two_simplex_sort_defined")(
            _dtype_code(a.dtype), _dtype_code(np.float64 if result == "double" else np.float32),
            _ptr(a), C.c_int64(m), C.c_int64(n), C.c_int64(int(p)), C.c_double(float(rhs)), _ptr(flags))
        if rc != 0:
            raise RuntimeError("two_simplex_sort_defined -> %d" % rc)
        return flags.astype(bool)


_cache = {}


def reference():
    if "ref" not in _cache:
        _cache["ref"] = Reference()
    return _cache["ref"]


def reference_accurate():
    if "acc" not in _cache:
        _cache["acc"] = ReferenceAccurate()
    return _cache["acc"]


def restatement():
    if "res" not in _cache:
        _cache["res"] = Restatement()
    return _cache["res"]


def have_reference():
    return os.path.exists(Reference.path)


def find_openblas():
    """An optimised CBLAS that ships inside this image (used for timing only)."""
    import glob
    import sys
    for sp in sys.path:
        folder = os.path.join(sp, "opencv_python_headless.libs")
        hits = glob.glob(os.path.join(folder, "libopenblas*.so*"))
        if hits:
            # its Fortran run-time lies beside it, outside the loader's search path: bring it
            # in first so that the dlopen of the BLAS resolves it
            try:
                for dep in ("libquadmath*.so*", "libgfortran*.so*"):
                    for f in glob.glob(os.path.join(folder, dep)):
                        C.CDLL(f, mode=C.RTLD_GLOBAL)
            except OSError:
                return None
            return hits[0]
    return None
