"""Pins the plain-C restatement (oracle/sdca_oracle.c) to the reference's own
headers (oracle/_ref): every prox operator on the regimes of the reference's
tests, and every objective's evaluation record on small random problems."""
import numpy as np
import pytest

from tests.util import (PROX_SINGLE, two_simplex_sort_defined, float_precision_ok, random_opts, regime, scaled_error,
                        stable_seed, tolerance)


@pytest.fixture(scope="module")
def port():
    from oracle import build_oracle, refapi
    build_oracle.build_restatement()
    return refapi.restatement()


@pytest.mark.parametrize("name", PROX_SINGLE + ["two_simplex", "two_simplex_sort"])
@pytest.mark.parametrize("dtype,precision", [(np.float64, "double"), (np.float32, "double"),
                                              (np.float32, "float")])
def test_prox_matches_reference(ref, port, name, dtype, precision):
    rng = np.random.default_rng(stable_seed("port", name, str(dtype), precision))
    for kind in ("normal", "pos", "neg", "mixed", "ties"):
        for m in (1, 2, 5, 33, 200):
            if name.startswith("two_simplex") and m < 2:
                continue
            a = regime(rng, 16, m, dtype, kind)
            kw = random_opts(rng, name, m)
            if name == "two_simplex_sort":
                a = a[two_simplex_sort_defined(ref, a, result=precision, **kw)]
                if len(a) == 0:
                    continue
            x_ref = ref.prox(name, a, result=precision, **kw)
            x = port.prox(name, a, result=precision, **kw)
            tol = tolerance(dtype, precision, m)
            if precision == "double":
                assert scaled_error(x, x_ref, a).max() <= tol, (name, kind, m, kw)
            else:
                ok, err = float_precision_ok(x, x_ref, ref.prox(name, a, result="double", **kw), a, tol)
                assert ok, (name, kind, m, kw, err)


def test_lambert_matches_reference(ref, port):
    for dtype in (np.float32, np.float64):
        x = np.linspace(-120, 120, 2001).astype(dtype)
        assert np.array_equal(port.lambert_w_exp(x), ref.lambert_w_exp(x))
        assert np.array_equal(port.prox("lambert_w_exp", x.reshape(1, -1)),
                              ref.prox("lambert_w_exp", x.reshape(1, -1)))


def random_problem(rng, n, d, m, dtype, multilabel):
    X = rng.standard_normal((n, d)).astype(dtype)
    if multilabel:
        labs, offs = [], [0]
        for _ in range(n):
            cnt = int(rng.integers(1, min(4, m)))
            labs.extend(sorted(rng.choice(m, size=cnt, replace=False).tolist()))
            offs.append(len(labs))
        labels, offsets = np.array(labs, dtype=np.int64), np.array(offs, dtype=np.int64)
        if labels.min() != 0:
            labels[0] = 0
    else:
        labels, offsets = rng.integers(0, m, n).astype(np.int64), None
        labels[0] = 0
    return X, labels, offsets


OBJECTIVES = ["l2_entropy", "l2_entropy_topk", "l2_hinge_topk", "l2_hinge_topk_smooth",
              "l2_topk_hinge", "l2_topk_hinge_smooth", "l2_multilabel_hinge",
              "l2_multilabel_hinge_smooth", "l2_multilabel_entropy"]


@pytest.mark.parametrize("objective", OBJECTIVES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("kernel", [False, True])
def test_eval_matches_reference(ref, port, objective, dtype, kernel):
    from oracle.refapi import MULTILABEL, OBJECTIVES as IDS
    rng = np.random.default_rng(stable_seed("eval", objective, str(dtype), kernel))
    n, d, m = 40, 12, 7
    ml = IDS[objective] in MULTILABEL
    X, labels, offsets = random_problem(rng, n, d, m, dtype, ml)
    # a feasible-looking dual point: a few SDCA epochs of the reference itself
    A = np.zeros((n, m), dtype=dtype); W = np.zeros((m, d), dtype=dtype)
    kw = dict(c=1.5, gamma=0.7, k=2)
    ref.fit(objective, X, A, labels, W=W, offsets=offsets, max_epoch=3, eval_epoch=10, **kw)
    if kernel:
        K = (X.astype(np.float64) @ X.astype(np.float64).T).astype(dtype)
        args = dict(kernel=True, offsets=offsets, **kw)
        r = ref.evaluate(objective, K, A.copy(), labels, **args)
        p = port.evaluate(objective, K, A.copy(), labels, **args)
    else:
        args = dict(W=W, offsets=offsets, **kw)
        r = ref.evaluate(objective, X, A.copy(), labels, **args)
        p = port.evaluate(objective, X, A.copy(), labels, **args)
    tol = 1e-12 if dtype == np.float64 else 1e-5
    for f in ("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer",
              "dual_regularizer", "rank_loss"):
        assert abs(r[f] - p[f]) <= tol * max(1, abs(r[f])), (f, r[f], p[f])
    assert np.allclose(r["accuracy"], p["accuracy"], atol=1e-12)
    # a held-out set: only the primal loss and the accuracy / rank loss
    Xt = X[:10] if not kernel else K[:10]
    lt = labels[:10] if not ml else labels[:offsets[10]]
    ot = None if not ml else offsets[:11]
    if kernel:
        rt = ref.evaluate(objective, Xt, A, lt, kernel=True, offsets=ot, is_train=False, **kw)
        pt = port.evaluate(objective, Xt, A, lt, kernel=True, offsets=ot, is_train=False, **kw)
    else:
        rt = ref.evaluate(objective, Xt, A, lt, W=W, offsets=ot, is_train=False, **kw)
        pt = port.evaluate(objective, Xt, A, lt, W=W, offsets=ot, is_train=False, **kw)
    assert abs(rt["primal_loss"] - pt["primal_loss"]) <= tol * max(1, abs(rt["primal_loss"]))
    assert np.allclose(rt["accuracy"], pt["accuracy"], atol=1e-12)
    assert abs(rt["rank_loss"] - pt["rank_loss"]) <= 1e-12


@pytest.mark.parametrize("n", [1, 2, 7, 1000, 46340, 46341, 50000])
def test_epoch_order_matches_reference(ref, port, n):
    assert np.array_equal(port.epoch_permutations(n, 3), ref.epoch_permutations(n, 3))


@pytest.mark.parametrize("objective", OBJECTIVES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("kernel", [False, True])
def test_fit_matches_reference(ref, port, objective, dtype, kernel):
    """The restated solver (steps of all nine objectives, epoch order, stopping rule)
    against solver::solve of the reference's headers."""
    from oracle.refapi import MULTILABEL, OBJECTIVES as IDS
    rng = np.random.default_rng(stable_seed("port-fit", objective, str(dtype), kernel))
    ml = IDS[objective] in MULTILABEL
    n, d, m = 60, 6, 6
    X, labels, offsets = random_problem(rng, n, d, m, dtype, ml)
    data = (X.astype(np.float64) @ X.astype(np.float64).T).astype(dtype) if kernel else X
    kw = dict(c=0.9, gamma=0.7, k=2, epsilon=1e-3, max_epoch=12, eval_epoch=2, offsets=offsets, kernel=kernel)
    A_ref = np.zeros((n, m), dtype=dtype); W_ref = np.zeros((m, d), dtype=dtype)
    A = np.zeros((n, m), dtype=dtype); W = np.zeros((m, d), dtype=dtype)
    r = ref.fit(objective, data, A_ref, labels, W=None if kernel else W_ref, **kw)
    p = port.fit(objective, data, A, labels, W=None if kernel else W, **kw)
    tol = 1e-10 if dtype == np.float64 else 2e-4
    assert p["status"] == r["status"] and p["epoch"] == r["epoch"]
    assert len(p["history"]) == len(r["history"])
    assert np.abs(A - A_ref).max() <= tol * max(1.0, np.abs(A_ref).max())
    if not kernel:
        assert np.abs(W - W_ref).max() <= tol * max(1.0, np.abs(W_ref).max()) * d
    assert np.abs(p["history"][:, :2] - r["history"][:, :2]).max() <= 10 * tol * max(1.0, np.abs(r["history"][:, :2]).max())


def test_fit_matches_golden(port):
    """The committed fits of the reference's solver (no reference tree needed)."""
    from tests.golden_util import fit_cases
    for c in fit_cases():
        A = np.zeros_like(c["A"]); W = np.zeros_like(c["W"])
        p = port.fit(c["objective"], c["data"], A, c["labels"], W=None if c["kernel"] else W,
                     kernel=c["kernel"], offsets=c["offsets"], c=c["c"], gamma=c["gamma"], k=c["k"],
                     epsilon=c["epsilon"], max_epoch=c["max_epoch"], eval_epoch=c["eval_epoch"])
        tol = 1e-10 if c["data"].dtype == np.float64 else 2e-4
        assert p["status"] == c["status"] and p["epoch"] == c["epoch"]
        assert np.abs(A - c["A"]).max() <= tol * max(1.0, np.abs(c["A"]).max())
