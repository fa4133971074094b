"""Generates tests/golden/*.npz from the reference's own headers.

Run where the reference tree is available (it builds oracle/_ref first):
    python tests/golden/make_golden.py          # everything
    python tests/golden/make_golden.py fit      # only fit_golden.npz
The vectors are small seeded inputs together with the outputs, thresholds and
evaluation records the reference produced for them; the tests load them without
needing the reference.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_oracle, refapi  # noqa: E402
from tests.util import PROX_SINGLE, random_opts, regime  # noqa: E402
from tests.test_oracle_restatement import OBJECTIVES, random_problem  # noqa: E402


HINGE = ("l2_hinge_topk", "l2_hinge_topk_smooth", "l2_topk_hinge", "l2_topk_hinge_smooth",
         "l2_entropy_topk", "l2_entropy")


def make_fit(ref):
    """Small fits by the reference's solver: inputs, final variables, the records
    of every evaluation, status and epoch count, and the order of the epochs."""
    rng = np.random.default_rng(20240919)
    out = {}
    idx = 0
    for objective in HINGE + ("l2_multilabel_hinge", "l2_multilabel_hinge_smooth", "l2_multilabel_entropy"):
        ml = refapi.OBJECTIVES[objective] in refapi.MULTILABEL
        for dtype in (np.float32, np.float64):
            for kernel in (False, True):
                n, d, m = 48, 6, 5
                X, labels, offsets = random_problem(rng, n, d, m, dtype, ml)
                data = (X.astype(np.float64) @ X.astype(np.float64).T).astype(dtype) if kernel else X
                A = np.zeros((n, m), dtype=dtype); W = np.zeros((m, d), dtype=dtype)
                kw = dict(c=0.8, gamma=0.6, k=2)
                r = ref.fit(objective, data, A, labels, W=None if kernel else W, kernel=kernel,
                            offsets=offsets, epsilon=1e-3, max_epoch=25, eval_epoch=2, **kw)
                key = "fit%03d" % idx
                idx += 1
                out[key + "_objective"] = np.array(objective)
                out[key + "_kernel"] = np.array(kernel)
                out[key + "_data"] = data
                out[key + "_labels"] = labels
                out[key + "_offsets"] = offsets if offsets is not None else np.zeros(0, dtype=np.int64)
                out[key + "_params"] = np.array([kw["c"], kw["gamma"], kw["k"], 1e-3, 25, 2])
                out[key + "_A"] = A
                out[key + "_W"] = W
                out[key + "_history"] = r["history"]
                out[key + "_status"] = np.array([r["status"], r["epoch"]])
    out["order_n50000_first64"] = ref.epoch_permutations(50000, 2)[:, :64]
    out["order_n1000"] = ref.epoch_permutations(1000, 3)
    np.savez_compressed(os.path.join(HERE, "fit_golden.npz"), **out)
    print("wrote", len(out), "fit arrays")


def main():
    build_oracle.build_reference()
    ref = refapi.reference()
    if sys.argv[1:] == ["fit"]:
        make_fit(ref)
        return
    rng = np.random.default_rng(20240607)
    out = {}
    idx = 0
    for name in PROX_SINGLE + ["two_simplex", "lambert_w_exp"]:
        for dtype in (np.float32, np.float64):
            for kind, m in (("normal", 40), ("ties", 64), ("mixed", 7)):
                a = regime(rng, 6, m, dtype, kind)
                if name == "lambert_w_exp":
                    a = (a * 12).astype(dtype)
                kw = random_opts(rng, name, m)
                key = "prox%03d" % idx
                idx += 1
                out[key + "_name"] = np.array(name)
                out[key + "_in"] = a
                out[key + "_opts"] = np.array([kw.get("lo", 0.0), kw.get("hi", 1.0), kw.get("rhs", 1.0),
                                               kw.get("rho", 1.0), kw.get("alpha", 1.0),
                                               kw.get("k", 1), kw.get("p", 1)], dtype=np.float64)
                out[key + "_out"] = ref.prox(name, a, **kw)
                if name != "lambert_w_exp":
                    th = ref.thresholds(name, a, **kw)
                    out[key + "_thr"] = np.stack([th["t"], th["lo"], th["hi"],
                                                  th["num_hi"].astype(np.float64),
                                                  th["num_mid"].astype(np.float64)], axis=1)
    np.savez_compressed(os.path.join(HERE, "prox_golden.npz"), **out)

    ev = {}
    idx = 0
    for objective in OBJECTIVES:
        for dtype in (np.float32, np.float64):
            for kernel in (False, True):
                ml = refapi.OBJECTIVES[objective] in refapi.MULTILABEL
                n, d, m = 24, 9, 6
                X, labels, offsets = random_problem(rng, n, d, m, dtype, ml)
                A = np.zeros((n, m), dtype=dtype); W = np.zeros((m, d), dtype=dtype)
                kw = dict(c=1.25, gamma=0.8, k=2)
                ref.fit(objective, X, A, labels, W=W, offsets=offsets, max_epoch=2, eval_epoch=10, **kw)
                if kernel:
                    K = (X.astype(np.float64) @ X.astype(np.float64).T).astype(dtype)
                    rec = ref.evaluate(objective, K, A.copy(), labels, kernel=True, offsets=offsets, **kw)
                    data = K
                else:
                    rec = ref.evaluate(objective, X, A.copy(), labels, W=W, offsets=offsets, **kw)
                    data = X
                key = "eval%03d" % idx
                idx += 1
                ev[key + "_objective"] = np.array(objective)
                ev[key + "_kernel"] = np.array(kernel)
                ev[key + "_data"] = data
                ev[key + "_A"] = A
                ev[key + "_W"] = W
                ev[key + "_labels"] = labels
                ev[key + "_offsets"] = offsets if offsets is not None else np.zeros(0, dtype=np.int64)
                ev[key + "_params"] = np.array([kw["c"], kw["gamma"], kw["k"]])
                ev[key + "_record"] = np.array([rec[f] for f in refapi.EVAL_FIELDS])
                ev[key + "_accuracy"] = rec["accuracy"]
    np.savez_compressed(os.path.join(HERE, "eval_golden.npz"), **ev)
    print("wrote", len(out), "prox arrays and", len(ev), "eval arrays")
    make_fit(ref)


if __name__ == "__main__":
    main()
