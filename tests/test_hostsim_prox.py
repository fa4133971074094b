"""Threshold logic of the CUDA sources, compiled for the host with one lane per
row (tests/hostsim), against the reference on the regimes of its own tests.
This checks the algorithms; the warp plumbing is covered by the gpu tests."""
import numpy as np
import pytest

from tests.util import float_precision_ok, stable_seed, PROX_SINGLE, random_opts, regime, scaled_error, tolerance, thresholds_agree, two_simplex_sort_defined


@pytest.mark.parametrize("name", PROX_SINGLE + ["two_simplex", "two_simplex_sort"])
@pytest.mark.parametrize("dtype,precision", [(np.float64, "double"), (np.float32, "double"),
                                              (np.float32, "float")])
def test_matches_reference(ref, hostsim, name, dtype, precision):
    rng = np.random.default_rng(stable_seed(name, str(dtype), precision))
    for kind in ("normal", "pos", "neg", "mixed", "ties"):
        for m in (1, 2, 3, 5, 33, 200):
            if name.startswith("two_simplex") and m < 2:
                continue
            a = regime(rng, 24, m, dtype, kind)
            kw = random_opts(rng, name, m)
            if name == "two_simplex_sort":
                a = a[two_simplex_sort_defined(ref, a, result=precision, **kw)]
                if len(a) == 0:
                    continue
            x_ref = ref.prox(name, a, result=precision, **kw)
            x, _ = hostsim.run(name, a, precision=precision, **kw)
            tol = tolerance(dtype, precision, m)
            if precision == "double":
                err = scaled_error(x, x_ref, a).max()
                assert err <= tol, (name, kind, m, kw, err)
            else:
                ok, err = float_precision_ok(x, x_ref, ref.prox(name, a, result="double", **kw), a, tol)
                assert ok, (name, kind, m, kw, err)


@pytest.mark.parametrize("name,kw,cols", [
    ("topk_simplex", dict(k=5, rhs=1.0), 1000), ("topk_cone", dict(k=5), 1000),
    ("knapsack_eq", dict(), 100), ("topk_entropy", dict(k=10), 200),
    ("entropy", dict(hi=0.1), 200)])
def test_thresholds_and_sets(ref, hostsim, name, kw, cols):
    rng = np.random.default_rng(17)
    for dtype in (np.float32, np.float64):
        a = regime(rng, 64, cols, dtype, "ties")
        x, thr = hostsim.run(name, a, **kw)
        rt = ref.thresholds(name, a, **kw)
        x_ref = ref.prox(name, a, **kw)
        tol = tolerance(dtype, "double", cols)
        assert scaled_error(x, x_ref, a).max() <= tol
        thresholds_agree(thr, rt, x, x_ref, a, tol)


def test_lambert(ref, hostsim):
    for dtype in (np.float32, np.float64):
        x = np.linspace(-120, 120, 4001).astype(dtype).reshape(1, -1)
        y, _ = hostsim.run("lambert_w_exp", x)
        y_ref = ref.prox("lambert_w_exp", x)
        assert np.array_equal(y, y_ref)


ACCURATE = ["knapsack_eq", "knapsack_le", "knapsack_le_biased", "topk_simplex", "topk_simplex_biased"]


@pytest.mark.parametrize("name", ACCURATE)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_accurate_math_matches_the_accurate_build(ref, ref_accurate, hostsim, name, dtype):
    """opts.accurate_math recomputes t from the final sets like the reference built with
    SDCA_ACCURATE_MATH (prox/knapsack_eq.h:87-106); compared with that build, and the
    recomputation really changes some thresholds against the default build."""
    rng = np.random.default_rng(stable_seed("accurate", name, str(dtype)))
    changed = 0
    for kind in ("normal", "pos", "neg", "mixed", "ties"):
        for m in (2, 3, 5, 33, 200):
            a = regime(rng, 24, m, dtype, kind)
            kw = random_opts(rng, name, m)
            x_ref = ref_accurate.prox(name, a, **kw)
            x, thr = hostsim.run(name, a, accurate_math=True, **kw)
            tol = tolerance(dtype, "double", m)
            assert scaled_error(x, x_ref, a).max() <= tol, (name, kind, m, kw)
            t_acc = ref_accurate.thresholds(name, a, **kw)["t"]
            t_def = ref.thresholds(name, a, **kw)["t"]
            changed += int((t_acc != t_def).sum())
            same = np.abs(thr["t"] - t_acc) <= tol * np.maximum(1, np.abs(t_acc))
            degenerate = ref_accurate.thresholds(name, a, **kw)["num_mid"] == 0
            # (the top-k operators report other thresholds for their special cases)
            assert name.startswith("topk") or (same | degenerate).all(), (name, kind, m, kw)
    assert changed > 0


@pytest.mark.parametrize("name", PROX_SINGLE + ["two_simplex", "two_simplex_sort"])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_nan_and_infinite_rows_end_with_a_defined_status(hostsim, name, dtype):
    """Rows with NaN or infinite entries: every search is bounded, so the call returns, and
    the thresholds entry point flags each such row (status bit 1: a threshold is not finite,
    or bit 0: the search ended on its default) or reports finite thresholds.  Clean rows in
    the same batch are unaffected.  (The reference asserts on such input, proxdef.h:112.)"""
    rng = np.random.default_rng(stable_seed("nonfinite", name, str(dtype)))
    for m in (2, 5, 33, 200):
        base = regime(rng, 12, m, dtype, "normal")
        kw = random_opts(rng, name, m)
        clean, thr_clean = hostsim.run(name, base, **kw)
        bad = base.copy()
        bad[1, 0] = np.nan
        bad[3, m // 2] = np.inf
        bad[5, m - 1] = -np.inf
        bad[7, :] = np.nan
        bad[9, 0] = np.inf; bad[9, m - 1] = -np.inf
        out, thr = hostsim.run(name, bad, **kw)          # returns: bounded termination
        per_row = 2 if name.startswith("two_simplex") else 1
        status = thr["status"].reshape(-1, per_row)
        assert set(np.unique(status)) <= {0, 1, 2, 3}
        finite_thr = np.isfinite(thr["t"]) & np.isfinite(thr["hi"]) & np.isfinite(thr["lo"])
        assert ((thr["status"] & 2) != 0)[~finite_thr].all()       # every non-finite record is flagged
        assert ((thr["status"] & 2) == 0)[finite_thr].all()
        for r in (0, 2, 4, 6, 8, 10, 11):
            assert np.array_equal(out[r], clean[r]) and (status[r] == thr_clean["status"].reshape(-1, per_row)[r]).all()
