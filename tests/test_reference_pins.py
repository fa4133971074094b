"""Pins the compiled reference (oracle/_ref) to the reference's own tests.

The reference ships no golden vectors; its prox tests are feasibility tests and
a few known-answer checks (test/prox/*.cpp).  They are restated here on the
library built from the reference's unmodified headers, so that everything else
in this suite can use that library as the oracle.
"""
import numpy as np
import pytest

from tests.util import regime

OMEGA = 0.5671432904097838729999686622103555497538157871865125081351310792230457930866


def test_lambert_omega(ref):
    # test/prox/lambert.cpp:144-157: lambert_w_exp(0) == Omega to one epsilon
    assert abs(ref.lambert_w_exp(np.array([0.0]))[0] - OMEGA) <= np.finfo(np.float64).eps
    assert abs(float(ref.lambert_w_exp(np.array([0.0], dtype=np.float32))[0]) - OMEGA) <= np.finfo(np.float32).eps


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_lambert_residuals(ref, dtype):
    # test/prox/lambert.cpp:5-87: |x - (w + log w)| < 4 eps max(1, x) for x > 0,
    # |e^x - w e^w| < 4 eps for x < 0
    rng = np.random.default_rng(1)
    eps = np.finfo(dtype).eps
    decades = range(-3, 3) if dtype == np.float32 else range(-6, 6)
    for p in decades:
        x = (rng.uniform(10.0 ** p, 10.0 ** (p + 1), 2000)).astype(dtype)
        w = ref.lambert_w_exp(x).astype(np.float64)
        assert (np.abs(x - (w + np.log(w))) < 4 * eps * np.maximum(1, x)).all()
        xn = -x
        wn = ref.lambert_w_exp(xn).astype(np.float64)
        assert (np.abs(np.exp(xn.astype(np.float64)) - wn * np.exp(wn)) < 4 * eps).all()


FEAS = [
    # name, options, kind of constraint on the sum, tolerance factor (test/prox/*.cpp)
    ("knapsack_eq", dict(lo=0.0, hi=1.0, rhs=1.0), "eq", 512),
    ("knapsack_le", dict(lo=0.0, hi=1.0, rhs=1.0), "le", 128),
    ("knapsack_le_biased", dict(lo=0.0, hi=1.0, rhs=1.0, rho=1.0), "le", 256),
    ("topk_simplex", dict(k=3, rhs=1.0), "le", 8),
    ("topk_simplex_biased", dict(k=3, rhs=1.0, rho=1.0), "le", 8),
    ("entropy", dict(hi=1.0, rhs=1.0), "eq", 8),
    ("entropy_norm", dict(hi=1.0, rhs=1.0), "eq", 8),
]


@pytest.mark.parametrize("name,opts,kind,factor", FEAS)
@pytest.mark.parametrize("reg", ["pos", "neg", "mixed"])
def test_reference_feasibility(ref, name, opts, kind, factor, reg):
    rng = np.random.default_rng(3)
    a = regime(rng, 50, 40, np.float64, reg)
    x = ref.prox(name, a, **opts)
    eps = np.finfo(np.float64).eps
    tol = factor * eps * np.maximum(1, np.abs(a).max(axis=1)) * a.shape[1]
    lo, hi, rhs = opts.get("lo", 0.0), opts.get("hi", np.inf), opts.get("rhs", 1.0)
    if name.startswith("topk_simplex"):
        hi = x.sum(axis=1, keepdims=True) / opts["k"]
    assert (x >= lo - 1e-300).all()
    assert (x <= hi + tol[:, None]).all()
    s = x.sum(axis=1)
    if kind == "eq":
        assert (np.abs(s - rhs) <= tol).all()
    else:
        assert (s <= rhs + tol).all()


def test_topk_cone_feasibility(ref):
    # test/prox/topk_cone.cpp: 0 <= x_i <= sum(x)/k
    rng = np.random.default_rng(5)
    for reg in ("pos", "neg", "mixed"):
        a = regime(rng, 50, 40, np.float64, reg)
        for k in (1, 3, 10):
            x = ref.prox("topk_cone", a, k=k)
            eps = np.finfo(np.float64).eps * np.maximum(1, np.abs(a).max(axis=1)) * a.shape[1]
            assert (x >= 0).all()
            assert (x <= x.sum(axis=1, keepdims=True) / k + eps[:, None]).all()


def test_topk_entropy_feasibility(ref):
    # test/prox/topk_entropy.cpp: 0 <= x_i <= s/k, s = sum(x) <= 1
    rng = np.random.default_rng(6)
    a = regime(rng, 50, 40, np.float64, "normal") * 3
    for k in (1, 4):
        x = ref.prox("topk_entropy", a, k=k)
        s = x.sum(axis=1)
        assert (s <= 1 + 1e-12).all() and (x >= 0).all()
        assert (x <= s[:, None] / k + 1e-12).all()


def test_two_simplex_degenerate_vector(ref):
    # test/prox/two_simplex.cpp:55-64 builds a vector whose two blocks must end
    # with equal sums; the property (sum x == sum y <= rhs, x, y >= 0) is checked
    a = np.array([[1e-6, 2.0, 3.0, -1.0, 0.5, 1e-9]])
    x = ref.prox("two_simplex", a, p=3, rhs=1.0)
    assert (x >= 0).all()
    assert abs(x[0, :3].sum() - x[0, 3:].sum()) < 1e-12
    assert x[0, :3].sum() <= 1 + 1e-12


def test_solver_toy_problem_converges(ref):
    # test/solver/solver.cpp:139-169: a separable toy problem must reach status
    # "solved" (2) with training accuracy 1 for every multiclass objective
    X = np.array([[0.0, 0.0, 1.0], [0.0, 1.0, 1.0], [1.0, 0.0, 1.0], [1.0, 1.0, 1.0]])
    labels = np.array([0, 1, 1, 1], dtype=np.int64)  # OR
    for obj in ("msvm", "msvm_smooth", "softmax", "topk_hinge_alpha", "l2_hinge_topk_smooth"):
        A = np.zeros((4, 2)); W = np.zeros((2, 3))
        r = ref.fit(obj, X, A, labels, W=W, c=10.0, gamma=1.0, k=1, epsilon=1e-9, eval_epoch=2)
        assert r["status"] == 2, obj
        assert r["accuracy"][0] == 1.0, obj
