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
                ("p", C.c_int64), ("precision", C.c_int32), ("accurate_math", C.c_int32)]


class Thresholds(C.Structure):
    _fields_ = [("t", C.c_double), ("lo", C.c_double), ("hi", C.c_double),
                ("num_hi", C.c_int32), ("num_mid", C.c_int32), ("status", C.c_int32),
                ("reserved", C.c_int32)]


THR_DTYPE = np.dtype([("t", "<f8"), ("lo", "<f8"), ("hi", "<f8"),
                      ("num_hi", "<i4"), ("num_mid", "<i4"), ("status", "<i4"), ("reserved", "<i4")])

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


def make_opts(lo=0.0, hi=1.0, rhs=1.0, rho=1.0, alpha=1.0, k=1, p=1, precision="double",
              accurate_math=False):
    prec = {"double": 0, "single": 1, "float": 1}.get(precision)
    if prec is None:
        # "long double" exists in the reference's front end but has no device type
        raise SdcabError(-8, "precision=%r" % (precision,))
    return ProxOpts(lo, hi, rhs, rho, alpha, int(k), int(p), prec, 1 if accurate_math else 0)


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


# ---------------------------------------------------------------- evaluation ----
class Objective(C.Structure):
    _fields_ = [("id", C.c_int32), ("precision", C.c_int32), ("c", C.c_double),
                ("gamma", C.c_double), ("k", C.c_int64)]


class EvalRecord(C.Structure):
    _fields_ = [("primal", C.c_double), ("dual", C.c_double), ("primal_loss", C.c_double),
                ("dual_loss", C.c_double), ("primal_regularizer", C.c_double),
                ("dual_regularizer", C.c_double), ("rank_loss", C.c_double),
                ("relative_gap", C.c_double)]


class Problem(C.Structure):
    _fields_ = [("input_kind", C.c_int32), ("is_train", C.c_int32), ("d", C.c_int64),
                ("n", C.c_int64), ("m", C.c_int64), ("a_row_offset", C.c_int64),
                ("x", C.c_void_p), ("a", C.c_void_p), ("w", C.c_void_p), ("w0", C.c_void_p),
                ("labels", C.c_void_p), ("offsets", C.c_void_p),
                ("include_primal_regularizer", C.c_int32), ("reserved", C.c_int32)]


RECORD_FIELDS = ("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer",
                 "dual_regularizer", "rank_loss", "relative_gap")


def make_objective(name, c=1.0, gamma=1.0, k=1, precision="double", from_name=None):
    """Objective by the names matsdca_fit accepts (src/matlab/mex_solve.cpp:643-715)."""
    o = Objective()
    if isinstance(name, int):
        # an objective class of the reference chosen directly (SDCAB_OBJ_* id)
        o.id = name; o.c = c; o.gamma = gamma; o.k = int(k)
        o.precision = {"double": 0, "single": 1, "float": 1}[precision]
        return o
    fn = from_name or lib().sdcab_objective_from_name
    _check(fn(name.encode(), C.c_double(c), C.c_double(gamma), C.c_int64(k), C.byref(o)),
           "sdcab_objective_from_name(%s)" % name)
    o.precision = {"double": 0, "single": 1, "float": 1}[precision]
    return o


def _ptr_of(x):
    if x is None:
        return None
    if _is_torch(x):
        return x.data_ptr()
    return x.ctypes.data


def make_problem(X, labels, A=None, W=None, W0=None, offsets=None, kernel=False, is_train=True,
                 a_row_offset=0, include_primal_regularizer=True):
    """X: (n, d) rows = examples (features) or kernel columns; A: (n_train, m); W: (m, d)."""
    n, d = X.shape
    m = A.shape[1] if A is not None else W.shape[0]
    p = Problem()
    p.input_kind = 1 if kernel else 0
    p.is_train = 1 if is_train else 0
    p.d = d; p.n = n; p.m = m; p.a_row_offset = a_row_offset
    p.x = _ptr_of(X); p.a = _ptr_of(A); p.w = _ptr_of(W); p.w0 = _ptr_of(W0)
    p.labels = _ptr_of(labels); p.offsets = _ptr_of(offsets)
    p.include_primal_regularizer = 1 if include_primal_regularizer else 0
    p._keep = (X, labels, A, W, W0, offsets)
    return p


def record_to_dict(rec, acc):
    out = {f: getattr(rec, f) for f in RECORD_FIELDS}
    out["accuracy"] = acc
    return out


def evaluate(objective, X, labels, A=None, W=None, W0=None, offsets=None, kernel=False,
             is_train=True, c=1.0, gamma=1.0, k=1, precision="double"):
    """Like one evaluate_dataset of the reference: returns the evaluation record.

    numpy inputs use the host-buffer entry point; torch CUDA tensors the device
    one (sums on the device, finish on the host)."""
    obj = objective if isinstance(objective, Objective) else make_objective(objective, c, gamma, k, precision)
    prob = make_problem(X, labels, A, W, W0, offsets, kernel, is_train)
    m = prob.m
    rec = EvalRecord()
    acc = np.zeros(m)
    if _is_torch(X):
        import torch
        sums = torch.zeros(8 + m, dtype=torch.float64, device=X.device)
        fn = getattr(lib(), "sdcab_eval_sums_%s_dev" % _suffix(str(X.dtype)))
        _check(fn(C.byref(obj), C.byref(prob), C.c_void_p(sums.data_ptr()), None, C.c_size_t(0),
                  _torch_stream()), "sdcab_eval_sums_dev")
        host = sums.cpu().numpy()
        _check(lib().sdcab_eval_finish(C.byref(obj), C.c_int64(m), host.ctypes.data_as(C.c_void_p),
                                       C.byref(rec), acc.ctypes.data_as(C.c_void_p)),
               "sdcab_eval_finish")
    else:
        fn = getattr(lib(), "sdcab_eval_%s" % _suffix(X.dtype.name))
        _check(fn(C.byref(obj), C.byref(prob), C.byref(rec), acc.ctypes.data_as(C.c_void_p)),
               "sdcab_eval")
    return record_to_dict(rec, acc)


def eval_sums_(objective, problem, sums, dtype_suffix, workspace=None, workspace_bytes=0):
    """Device sums of one shard (torch tensors inside ``problem``); for sharded runs."""
    fn = getattr(lib(), "sdcab_eval_sums_%s_dev" % dtype_suffix)
    _check(fn(C.byref(objective), C.byref(problem), C.c_void_p(sums.data_ptr()),
              C.c_void_p(workspace.data_ptr()) if workspace is not None else None,
              C.c_size_t(workspace_bytes), _torch_stream()), "sdcab_eval_sums_dev")
    return sums


def eval_finish(objective, m, sums_host):
    rec = EvalRecord()
    acc = np.zeros(m)
    sums_host = np.ascontiguousarray(sums_host, dtype=np.float64)
    _check(lib().sdcab_eval_finish(C.byref(objective), C.c_int64(m),
                                   sums_host.ctypes.data_as(C.c_void_p), C.byref(rec),
                                   acc.ctypes.data_as(C.c_void_p)), "sdcab_eval_finish")
    return record_to_dict(rec, acc)


# ---- fit -----------------------------------------------------------------------

class FitCriteria(C.Structure):
    _fields_ = [("epsilon", C.c_double), ("max_epoch", C.c_int64), ("eval_epoch", C.c_int64),
                ("eval_on_start", C.c_int32), ("recompute_primal", C.c_int32),
                ("max_cpu_time", C.c_double), ("max_wall_time", C.c_double)]


class FitResult(C.Structure):
    _fields_ = [("status", C.c_int32), ("reserved", C.c_int32), ("epoch", C.c_int64),
                ("num_evals", C.c_int64), ("solve_seconds", C.c_double),
                ("eval_seconds", C.c_double), ("cpu_seconds", C.c_double),
                ("wall_seconds", C.c_double)]


class FitHistory(C.Structure):
    _fields_ = [("cap", C.c_int64), ("num_tests", C.c_int64), ("tests", C.c_void_p),
                ("train", C.c_void_p), ("train_accuracy", C.c_void_p), ("epoch", C.c_void_p),
                ("wall_seconds", C.c_void_p), ("test", C.c_void_p), ("test_accuracy", C.c_void_p)]


class Dataset(C.Structure):
    _fields_ = [("n", C.c_int64), ("x", C.c_void_p), ("labels", C.c_void_p), ("offsets", C.c_void_p)]


class TrainOptions(C.Structure):
    _fields_ = [("objective", C.c_char_p), ("c", C.c_double), ("gamma", C.c_double), ("k", C.c_int64),
                ("is_dual", C.c_int32), ("precision", C.c_int32), ("criteria", FitCriteria),
                ("num_dimensions", C.c_int64), ("num_classes", C.c_int64), ("W0", C.c_void_p),
                ("warm_start", C.c_int32), ("reserved", C.c_int32)]


class Model(C.Structure):
    _fields_ = [("A", C.c_void_p), ("W", C.c_void_p), ("num_dimensions", C.c_int64),
                ("num_examples", C.c_int64), ("num_classes", C.c_int64), ("is_dual", C.c_int32),
                ("objective_id", C.c_int32), ("objective", C.c_char * 40), ("c", C.c_double),
                ("gamma", C.c_double), ("k", C.c_int64), ("criteria", FitCriteria),
                ("status", C.c_int32), ("data_precision", C.c_int32), ("precision", C.c_int32),
                ("labels_one_based", C.c_int32), ("epoch", C.c_int64), ("cpu_time", C.c_double),
                ("wall_time", C.c_double), ("solve_time", C.c_double), ("eval_time", C.c_double),
                ("relative_gap", C.c_double), ("num_evals", C.c_int64), ("history", FitHistory)]


class _HistoryBuffers:
    """Host arrays behind a FitHistory (kept alive with it)."""

    def __init__(self, cap, m, num_tests):
        self.cap, self.m, self.num_tests = cap, m, num_tests
        self.train = (EvalRecord * cap)()
        self.train_accuracy = np.zeros((cap, m))
        self.epoch = np.zeros(cap, dtype=np.int64)
        self.wall = np.zeros(cap)
        self.test = (EvalRecord * max(1, cap * num_tests))()
        self.test_accuracy = np.zeros((cap, max(1, num_tests), m))

    def fill(self, h):
        h.cap = self.cap; h.num_tests = self.num_tests
        h.train = C.cast(self.train, C.c_void_p)
        h.train_accuracy = self.train_accuracy.ctypes.data
        h.epoch = self.epoch.ctypes.data
        h.wall_seconds = self.wall.ctypes.data
        h.test = C.cast(self.test, C.c_void_p)
        h.test_accuracy = self.test_accuracy.ctypes.data

    def to_dict(self, num_evals):
        n = min(num_evals, self.cap)
        out = dict(
            train=[{f: getattr(self.train[i], f) for f in RECORD_FIELDS} for i in range(n)],
            train_accuracy=self.train_accuracy[:n].copy(), epoch=self.epoch[:n].copy(),
            wall_seconds=self.wall[:n].copy(), tests=[])
        for t in range(self.num_tests):
            recs = [self.test[i * self.num_tests + t] for i in range(n)]
            out["tests"].append(dict(primal_loss=np.array([r.primal_loss for r in recs]),
                                     rank_loss=np.array([r.rank_loss for r in recs]),
                                     accuracy=self.test_accuracy[:n, t].copy()))
        return out


FIT_STATUS = ("none", "solving", "solved", "no_progress", "max_epoch", "max_cpu_time",
              "max_wall_time", "failed")


def fit_result_to_dict(res, evals):
    count = min(res.num_evals, len(evals))
    return dict(status=FIT_STATUS[res.status], status_code=res.status, epoch=res.epoch,
                num_evals=res.num_evals, solve_seconds=res.solve_seconds,
                eval_seconds=res.eval_seconds, cpu_seconds=res.cpu_seconds,
                wall_seconds=res.wall_seconds,
                history=[{f: getattr(evals[i], f) for f in RECORD_FIELDS} for i in range(count)])


def epoch_permutations(n, num_epochs):
    """Example order of the reference's solver for its first ``num_epochs`` epochs."""
    perm = np.zeros((num_epochs, n), dtype=np.int64)
    _check(lib().sdcab_epoch_permutations(C.c_int64(n), C.c_int64(num_epochs),
                                          perm.ctypes.data_as(C.c_void_p)),
           "sdcab_epoch_permutations")
    return perm


def fit_(objective, X, labels, A, W=None, kernel=False, c=1.0, gamma=0.0, k=1,
         precision="double", epsilon=1e-3, max_epoch=1000, eval_epoch=10, eval_on_start=False,
         permutations=None, offsets=None, recompute_primal=False, W0=None,
         max_cpu_time=0.0, max_wall_time=0.0, tests=None):
    """SDCA fit, in place on ``A`` (n x m) and ``W`` (m x d): torch CUDA tensors use the
    device entry point, numpy arrays the host-buffer one (copies inside).

    Mirrors ``matsdca_fit``'s stopping options (src/matlab/mex_solve.cpp:505-528 of the
    reference); returns status, epochs and the evaluation records.  ``recompute_primal``
    rebuilds W from A before every evaluation (features only), which the reference does
    when it is compiled with SDCA_ACCURATE_MATH."""
    obj = objective if isinstance(objective, Objective) else make_objective(objective, c, gamma, k, precision)
    prob = make_problem(X, labels, A, W, W0, offsets, kernel, True)
    crit = FitCriteria(epsilon, max_epoch, eval_epoch, 1 if eval_on_start else 0,
                       1 if recompute_primal else 0, max_cpu_time, max_wall_time)
    cap = int(max_epoch) + 4
    evals = (EvalRecord * cap)()
    res = FitResult()
    perm = None
    if permutations is not None:
        perm = np.ascontiguousarray(permutations, dtype=np.int64)
        if perm.size < max_epoch * X.shape[0]:
            raise SdcabError(-1, "fit_: permutations must hold max_epoch * n indices")
    perm_ptr = perm.ctypes.data_as(C.c_void_p) if perm is not None else None
    if tests is not None:
        # held-out sets as (X, labels[, offsets]) tuples of the same kind as the training data:
        # evaluated after every evaluation of the training set
        m = prob.m
        bufs = _HistoryBuffers(cap, m, len(tests))
        tprobs = (Problem * max(1, len(tests)))()
        keep = []
        for i, t in enumerate(tests):
            tp = make_problem(t[0], t[1], A, W, None, t[2] if len(t) > 2 else None, kernel, False)
            keep.append(tp)
            tprobs[i] = tp
        hist = FitHistory()
        bufs.fill(hist)
        hist.tests = C.cast(tprobs, C.c_void_p)
        dev = _is_torch(X)
        name = "sdcab_fit_history_%s%s" % (_suffix(str(X.dtype) if dev else X.dtype.name), "_dev" if dev else "")
        args = [C.byref(obj), C.byref(prob), C.byref(crit), perm_ptr, C.byref(hist), C.byref(res)]
        if dev:
            args.append(_torch_stream())
        _check(getattr(lib(), name)(*args), name)
        out = dict(status=FIT_STATUS[res.status], status_code=res.status, epoch=res.epoch,
                   num_evals=res.num_evals, solve_seconds=res.solve_seconds,
                   eval_seconds=res.eval_seconds, cpu_seconds=res.cpu_seconds,
                   wall_seconds=res.wall_seconds)
        h = bufs.to_dict(res.num_evals)
        out["history"] = h["train"]
        out.update(train_accuracy=h["train_accuracy"], eval_epoch=h["epoch"], eval_wall_seconds=h["wall_seconds"],
                   tests=h["tests"])
        return out
    if _is_torch(X):
        fn = getattr(lib(), "sdcab_fit_%s_dev" % _suffix(str(X.dtype)))
        _check(fn(C.byref(obj), C.byref(prob), C.byref(crit), perm_ptr, evals, C.c_int64(cap),
                  C.byref(res), _torch_stream()), "sdcab_fit_dev")
    else:
        fn = getattr(lib(), "sdcab_fit_%s" % _suffix(X.dtype.name))
        _check(fn(C.byref(obj), C.byref(prob), C.byref(crit), perm_ptr, evals, C.c_int64(cap),
                  C.byref(res)), "sdcab_fit")
    return fit_result_to_dict(res, evals)


def train(data, labels, objective=None, c=1.0, gamma=1.0, k=1, is_dual=False, precision="double",
          epsilon=1e-3, max_epoch=1000, eval_epoch=10, eval_on_start=False, max_cpu_time=0.0,
          max_wall_time=0.0, A=None, W=None, W0=None, offsets=None, num_classes=0):
    """``matsdca_fit(data, labels, opts)`` on numpy arrays (src/matlab/mex_solve.cpp:473-620 of
    the reference): ``data`` is one (n, d) feature matrix -- or (n, n_train) Gram columns with
    ``is_dual`` -- or a list of them, the first for training, the others evaluated only;
    ``labels`` (and ``offsets`` for multilabel objectives) likewise.  Labels may be 0-based or
    1-based.  ``A`` / ``W`` given: warm start.  Returns the model as a dict."""
    sets = data if isinstance(data, (list, tuple)) else [data]
    labs = labels if isinstance(labels, (list, tuple)) else [labels]
    offs = offsets if isinstance(offsets, (list, tuple)) else [offsets] * len(sets)
    dtype = sets[0].dtype
    n = sets[0].shape[0]
    d = sets[0].shape[1]
    ds = (Dataset * len(sets))()
    keep = []
    for i, (x, l, o) in enumerate(zip(sets, labs, offs)):
        x = np.ascontiguousarray(x, dtype=dtype); l = np.ascontiguousarray(l, dtype=np.int64)
        keep += [x, l]
        ds[i].n = x.shape[0]; ds[i].x = x.ctypes.data; ds[i].labels = l.ctypes.data
        if o is not None:
            o = np.ascontiguousarray(o, dtype=np.int64); keep.append(o)
            ds[i].offsets = o.ctypes.data
    opts = TrainOptions()
    lib().sdcab_train_options_default(C.byref(opts))
    if objective is not None:
        opts.objective = objective.encode()
    opts.c = c; opts.gamma = gamma; opts.k = k; opts.is_dual = 1 if is_dual else 0
    opts.precision = {"double": 0, "single": 1, "float": 1}[precision]
    opts.criteria = FitCriteria(epsilon, max_epoch, eval_epoch, 1 if eval_on_start else 0, 0,
                                max_cpu_time, max_wall_time)
    opts.num_dimensions = d; opts.num_classes = num_classes
    if W0 is not None:
        W0 = np.ascontiguousarray(W0, dtype=dtype); opts.W0 = W0.ctypes.data
    l0 = np.asarray(labs[0])
    m = num_classes or int(l0.max() - min(1, l0.min()) + 1)
    opts.warm_start = 1 if A is not None else 0
    A = np.zeros((n, m), dtype=dtype) if A is None else np.ascontiguousarray(A, dtype=dtype)
    if not is_dual:
        W = np.zeros((m, d), dtype=dtype) if W is None else np.ascontiguousarray(W, dtype=dtype)
    model = Model()
    model.A = A.ctypes.data
    model.W = W.ctypes.data if W is not None else None
    cap = int(max_epoch) + 4
    bufs = _HistoryBuffers(cap, m, len(sets) - 1)
    bufs.fill(model.history)
    fn = getattr(lib(), "sdcab_train_%s" % _suffix(dtype.name))
    _check(fn(ds, C.c_int64(len(sets)), C.byref(opts), C.byref(model)), "sdcab_train")
    h = bufs.to_dict(model.num_evals)
    return dict(A=A, W=W, num_dimensions=model.num_dimensions, num_examples=model.num_examples,
                num_classes=model.num_classes, is_dual=bool(model.is_dual),
                objective=model.objective.decode(), objective_id=model.objective_id, c=model.c,
                k=model.k, gamma=model.gamma, status=FIT_STATUS[model.status], epoch=model.epoch,
                cpu_time=model.cpu_time, wall_time=model.wall_time, relative_gap=model.relative_gap,
                labels_one_based=bool(model.labels_one_based), num_evals=model.num_evals,
                train=h["train"], train_accuracy=h["train_accuracy"], eval_epoch=h["epoch"],
                tests=h["tests"])


class Comm:
    """The ranks of a sharded evaluation (``sdcab_comm``): NCCL behind the C ABI."""

    ID_BYTES = 128

    def __init__(self, handle):
        self.handle = handle

    @staticmethod
    def unique_id():
        buf = C.create_string_buffer(Comm.ID_BYTES)
        _check_comm(lib().sdcab_comm_unique_id(buf), "sdcab_comm_unique_id")
        return buf.raw

    @staticmethod
    def create(nranks, rank, unique_id):
        h = C.c_void_p()
        _check_comm(lib().sdcab_comm_create(C.byref(h), int(nranks), int(rank), unique_id), "sdcab_comm_create")
        return Comm(h)

    def allreduce_(self, t):
        """In-place sum of a float32 / float64 torch CUDA tensor over the ranks."""
        fn = getattr(lib(), "sdcab_comm_allreduce_%s" % _suffix(str(t.dtype)))
        _check_comm(fn(self.handle, C.c_void_p(t.data_ptr()), C.c_int64(t.numel()), _torch_stream()),
                    "sdcab_comm_allreduce")
        return t

    def eval_sums_(self, objective, problem, sums, dtype_suffix, workspace=None, workspace_bytes=0):
        """This rank's shard evaluated and the sums added over the ranks."""
        fn = getattr(lib(), "sdcab_eval_sums_sharded_%s_dev" % dtype_suffix)
        _check_comm(fn(C.byref(objective), C.byref(problem), C.c_void_p(sums.data_ptr()),
                       C.c_void_p(workspace.data_ptr()) if workspace is not None else None,
                       C.c_size_t(workspace_bytes), self.handle, _torch_stream()),
                    "sdcab_eval_sums_sharded_dev")
        return sums

    def destroy(self):
        if self.handle:
            lib().sdcab_comm_destroy(self.handle)
            self.handle = None


def _check_comm(rc, where):
    if rc == -24:
        lib().sdcab_comm_last_error.restype = C.c_char_p
        raise SdcabError(rc, where + ": " + lib().sdcab_comm_last_error().decode())
    _check(rc, where)


def test_set(name, value):
    """Switches for the library's own tests (``sdcab_test_set``)."""
    _check(lib().sdcab_test_set(name.encode(), C.c_int64(int(value))), "sdcab_test_set(%s)" % name)


def primal_from_dual(X, A, W0=None, out=None):
    """W = [W0 +] X A' on the device (eval_recompute_primal of the reference,
    include/sdca/solver/eval/core.h:148-182).  Torch CUDA tensors in the layouts of
    ``fit_``: X is n x d (rows = examples), A is n x m, W0 / the result m x d."""
    import torch
    n, d = X.shape
    m = A.shape[1]
    if A.shape[0] != n or X.dtype != A.dtype or not (X.is_contiguous() and A.is_contiguous()):
        raise SdcabError(-1, "primal_from_dual: X (n x d) and A (n x m), contiguous, same dtype")
    if W0 is not None and (tuple(W0.shape) != (m, d) or W0.dtype != X.dtype or not W0.is_contiguous()):
        raise SdcabError(-1, "primal_from_dual: W0 must be m x d")
    if out is None:
        out = torch.empty((m, d), dtype=X.dtype, device=X.device)
    fn = getattr(lib(), "sdcab_primal_from_dual_%s_dev" % _suffix(str(X.dtype)))
    _check(fn(C.c_void_p(X.data_ptr()), C.c_void_p(A.data_ptr()),
              C.c_void_p(W0.data_ptr()) if W0 is not None else None, C.c_void_p(out.data_ptr()),
              C.c_int64(d), C.c_int64(m), C.c_int64(n), _torch_stream()), "sdcab_primal_from_dual")
    return out
