"""Per-example loss / conjugate code of the CUDA sources (losses.cuh), compiled
for the host with one lane per example, against the reference's evaluation
records and the committed golden records."""
import numpy as np
import pytest

from tests.golden_util import eval_cases
from tests.test_oracle_restatement import OBJECTIVES, random_problem
from tests.util import stable_seed

FIELDS = ("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer",
          "dual_regularizer", "rank_loss")


def compare(rec, ref_rec, tol):
    for f in FIELDS:
        assert abs(rec[f] - ref_rec[f]) <= tol * max(1, abs(ref_rec[f])), (f, rec[f], ref_rec[f])
    assert np.allclose(rec["accuracy"], ref_rec["accuracy"], atol=1e-12)


@pytest.mark.parametrize("objective", OBJECTIVES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("kernel", [False, True])
def test_eval_matches_reference(ref, hostsim, objective, dtype, kernel):
    from oracle.refapi import MULTILABEL, OBJECTIVES as IDS
    rng = np.random.default_rng(stable_seed("hostsim-eval", objective, str(dtype), kernel))
    ml = IDS[objective] in MULTILABEL
    for n, d, m, k in ((40, 12, 7, 2), (33, 5, 40, 5), (9, 3, 2, 1)):
        X, labels, offsets = random_problem(rng, n, d, m, dtype, ml)
        if ml and m == 2:
            continue
        A = np.zeros((n, m), dtype=dtype); W = np.zeros((m, d), dtype=dtype)
        kw = dict(c=1.5, gamma=0.7, k=k)
        ref.fit(objective, X, A, labels, W=W, offsets=offsets, max_epoch=3, eval_epoch=10, **kw)
        tol = 1e-12 if dtype == np.float64 else 1e-5
        if kernel:
            K = (X.astype(np.float64) @ X.astype(np.float64).T).astype(dtype)
            r = ref.evaluate(objective, K, A.copy(), labels, kernel=True, offsets=offsets, **kw)
            h = hostsim.evaluate(IDS[objective], K, labels, A=A, offsets=offsets, kernel=True, **kw)
        else:
            r = ref.evaluate(objective, X, A.copy(), labels, W=W, offsets=offsets, **kw)
            h = hostsim.evaluate(IDS[objective], X, labels, A=A, W=W, offsets=offsets, **kw)
        compare(h, r, tol)


def test_golden_eval_records(hostsim):
    from oracle.refapi import EVAL_FIELDS, OBJECTIVES as IDS
    for c in eval_cases():
        kw = dict(c=c["c"], gamma=c["gamma"], k=c["k"], offsets=c["offsets"])
        if c["kernel"]:
            h = hostsim.evaluate(IDS[c["objective"]], c["data"], c["labels"], A=c["A"], kernel=True, **kw)
        else:
            h = hostsim.evaluate(IDS[c["objective"]], c["data"], c["labels"], A=c["A"], W=c["W"], **kw)
        tol = 1e-12 if c["data"].dtype == np.float64 else 1e-5
        ref_rec = {f: c["record"][i] for i, f in enumerate(EVAL_FIELDS)}
        ref_rec["accuracy"] = c["accuracy"]
        compare(h, ref_rec, tol)


def test_objective_names(hostsim):
    from libsdca_b200 import binding as b
    fn = hostsim.lib.sdcab_hostsim_objective_from_name
    assert b.make_objective("msvm", from_name=fn).id == 4
    assert b.make_objective("msvm_smooth", from_name=fn).id == 5
    assert b.make_objective("topk_hinge_alpha", gamma=0.0, k=3, from_name=fn).id == 2
    assert b.make_objective("topk_hinge_alpha", gamma=1.0, k=3, from_name=fn).id == 3
    assert b.make_objective("l2_topk_hinge", gamma=0.0, k=3, from_name=fn).id == 4
    assert b.make_objective("softmax", from_name=fn).id == 0
    assert b.make_objective("mlsoftmax", from_name=fn).id == 8
    o = b.Objective()
    assert fn(b"msvm", C_double(1.0), C_double(1.0), 2, o) == -2   # k must be 1
    assert fn(b"nope", C_double(1.0), C_double(1.0), 1, o) == -7
    assert fn(b"softmax", C_double(0.0), C_double(1.0), 1, o) == -2  # c > 0


from ctypes import c_double as C_double  # noqa: E402
