"""Builds and loads the test-only single-lane host build of the threshold code."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libsdcab_hostsim.so")
CSRC = os.path.join(HERE, "..", "..", "libsdca_b200", "csrc")


def build():
    deps = [os.path.join(HERE, "hostsim.cpp")] + [
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    if os.path.exists(SO) and all(os.path.getmtime(d) <= os.path.getmtime(SO) for d in deps):
        return SO
    subprocess.run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-x", "c++",
                    os.path.join(HERE, "hostsim.cpp"), "-o", SO], check=True)
    return SO


class HostSim:
    def __init__(self):
        self.lib = C.CDLL(build())

    def run(self, name, a, precision="double", **kw):
        """Returns (prox output, thresholds structured array)."""
        from libsdca_b200.binding import THR_DTYPE, make_opts
        a = np.array(a, order="C", copy=True)
        n, m = a.shape
        o = make_opts(precision=precision, **kw)
        two = name.startswith("two_")
        thr = np.zeros(2 * n if two else n, dtype=THR_DTYPE)
        rc = self.lib.sdcab_hostsim_prox(
            name.encode(), 0 if a.dtype == np.float32 else 1, a.ctypes.data_as(C.c_void_p),
            C.c_int64(m), C.c_int64(n), C.byref(o), thr.ctypes.data_as(C.c_void_p), 1)
        assert rc == 0, rc
        return a, thr


    def evaluate(self, objective, X, labels, A=None, W=None, W0=None, offsets=None, kernel=False,
                 is_train=True, c=1.0, gamma=1.0, k=1, precision="double"):
        from libsdca_b200 import binding as b
        obj = b.make_objective(objective, c, gamma, k, precision,
                               from_name=self.lib.sdcab_hostsim_objective_from_name)
        prob = b.make_problem(X, labels, A, W, W0, offsets, kernel, is_train)
        m = prob.m
        sums = np.zeros(8 + m)
        rc = self.lib.sdcab_hostsim_eval(C.byref(obj), C.byref(prob),
                                         0 if X.dtype == np.float32 else 1,
                                         sums.ctypes.data_as(C.c_void_p))
        assert rc == 0, rc
        rec = b.EvalRecord(); acc = np.zeros(m)
        rc = self.lib.sdcab_hostsim_eval_finish(C.byref(obj), C.c_int64(m),
                                                sums.ctypes.data_as(C.c_void_p), C.byref(rec),
                                                acc.ctypes.data_as(C.c_void_p))
        assert rc == 0, rc
        return b.record_to_dict(rec, acc)

    def fit(self, objective, X, labels, A, W=None, kernel=False, c=1.0, gamma=0.0, k=1,
            precision="double", epsilon=1e-3, max_epoch=100, eval_epoch=1, eval_on_start=False,
            permutations=None, offsets=None):
        """Runs the fit in place on A (and W); returns status, epoch and the records."""
        from libsdca_b200 import binding as b
        obj = b.make_objective(objective, c, gamma, k, precision,
                               from_name=self.lib.sdcab_hostsim_objective_from_name)
        prob = b.make_problem(X, labels, A, W, None, offsets, kernel, True)
        crit = b.FitCriteria(epsilon, max_epoch, eval_epoch, 1 if eval_on_start else 0, 0)
        cap = max_epoch + 4
        evals = (b.EvalRecord * cap)()
        res = b.FitResult()
        perm = None
        if permutations is not None:
            perm = np.ascontiguousarray(permutations, dtype=np.int64)
        rc = self.lib.sdcab_hostsim_fit(
            C.byref(obj), C.byref(prob), 0 if X.dtype == np.float32 else 1, C.byref(crit),
            perm.ctypes.data_as(C.c_void_p) if perm is not None else None, evals, C.c_int64(cap),
            C.byref(res))
        assert rc == 0, rc
        return b.fit_result_to_dict(res, evals)

    def epoch_permutations(self, n, epochs):
        perm = np.zeros((epochs, n), dtype=np.int64)
        self.lib.sdcab_hostsim_epoch_permutations(C.c_int64(n), C.c_int64(epochs),
                                                  perm.ctypes.data_as(C.c_void_p))
        return perm


def load():
    return HostSim()
