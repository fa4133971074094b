"""The SDCA step of the CUDA sources (update_core.cuh), the epoch order and the
stopping rule (fit_host.h), compiled for the host with one lane, against the
reference's solver on the same problems."""
import numpy as np
import pytest

from libsdca_b200.synth import kernel_problem
from tests.test_oracle_restatement import random_problem
from tests.util import stable_seed

HINGE = ("l2_hinge_topk", "l2_hinge_topk_smooth", "l2_topk_hinge", "l2_topk_hinge_smooth",
         "l2_entropy_topk", "l2_entropy")
REF_STATUS = ("none", "solving", "solved", "no_progress", "max_epoch", "max_cpu_time",
              "max_wall_time", "failed")


@pytest.mark.parametrize("n", [1, 2, 3, 10, 101, 1000, 46340, 46341, 50000])
def test_epoch_order_matches_std_shuffle(ref, hostsim, n):
    epochs = 3
    assert np.array_equal(hostsim.epoch_permutations(n, epochs), ref.epoch_permutations(n, epochs))


def check_fit(ref, hostsim, objective, data, labels, kernel, dtype, tol, **kw):
    from oracle.refapi import OBJECTIVES as IDS
    n = data.shape[0]
    m = int(labels.max()) + 1 if kw.get("m") is None else kw.pop("m")
    d = data.shape[1]
    fit_kw = dict(epsilon=kw.pop("epsilon", 1e-3), max_epoch=kw.pop("max_epoch", 30),
                  eval_epoch=kw.pop("eval_epoch", 1), eval_on_start=kw.pop("eval_on_start", False))
    A_ref = np.zeros((n, m), dtype=dtype); W_ref = np.zeros((m, d), dtype=dtype)
    A = np.zeros((n, m), dtype=dtype); W = np.zeros((m, d), dtype=dtype)
    r = ref.fit(objective, data, A_ref, labels, W=None if kernel else W_ref, kernel=kernel,
                **fit_kw, **kw)
    h = hostsim.fit(IDS[objective], data, labels, A, W=None if kernel else W, kernel=kernel,
                    **fit_kw, **kw)
    assert h["status"] == REF_STATUS[r["status"]], (h["status"], r["status"])
    assert h["epoch"] == r["epoch"]
    assert h["num_evals"] == len(r["history"])
    scale = max(1.0, np.abs(A_ref).max())
    assert np.abs(A - A_ref).max() <= tol * scale, np.abs(A - A_ref).max()
    if not kernel:
        assert np.abs(W - W_ref).max() <= tol * max(1.0, np.abs(W_ref).max()) * d
    last, rlast = h["history"][-1], r["history"][-1]
    for i, f in enumerate(("primal", "dual")):
        assert abs(last[f] - rlast[i]) <= 10 * tol * max(1.0, abs(rlast[i])), (f, last[f], rlast[i])


@pytest.mark.parametrize("objective", HINGE)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_kernel_fit_matches_reference(ref, hostsim, objective, dtype):
    K, labels = kernel_problem(n=120, dim=8, m=6, seed=stable_seed("fit", objective) % 1000, dtype=dtype)
    tol = 1e-9 if dtype == np.float64 else 2e-4
    for k in (1, 2):
        check_fit(ref, hostsim, objective, K, labels, True, dtype, tol, m=6, c=1.0, gamma=0.5, k=k)


@pytest.mark.parametrize("objective", HINGE)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_feature_fit_matches_reference(ref, hostsim, objective, dtype):
    rng = np.random.default_rng(stable_seed("fit-features", objective, str(dtype)))
    X, labels, _ = random_problem(rng, 90, 7, 5, dtype, False)
    tol = 1e-9 if dtype == np.float64 else 2e-4
    check_fit(ref, hostsim, objective, X, labels, False, dtype, tol, m=5, c=0.7, gamma=1.0, k=2,
              max_epoch=12, eval_epoch=3)


@pytest.mark.parametrize("objective", ["l2_multilabel_hinge", "l2_multilabel_hinge_smooth",
                                       "l2_multilabel_entropy"])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("kernel", [False, True])
def test_multilabel_fit_matches_reference(ref, hostsim, objective, dtype, kernel):
    from oracle.refapi import OBJECTIVES as IDS
    rng = np.random.default_rng(stable_seed("fit-multilabel", objective, str(dtype), kernel))
    n, d, m = 70, 6, 7
    X, labels, offsets = random_problem(rng, n, d, m, dtype, True)
    data = (X.astype(np.float64) @ X.astype(np.float64).T).astype(dtype) if kernel else X
    tol = 1e-9 if dtype == np.float64 else 2e-4
    kw = dict(c=0.9, gamma=0.7, k=1, epsilon=1e-3, max_epoch=15, eval_epoch=2)
    A_ref = np.zeros((n, m), dtype=dtype); W_ref = np.zeros((m, d), dtype=dtype)
    A = np.zeros((n, m), dtype=dtype); W = np.zeros((m, d), dtype=dtype)
    r = ref.fit(objective, data, A_ref, labels, W=None if kernel else W_ref, kernel=kernel,
                offsets=offsets, **kw)
    h = hostsim.fit(IDS[objective], data, labels, A, W=None if kernel else W, kernel=kernel,
                    offsets=offsets, **kw)
    assert h["status"] == REF_STATUS[r["status"]] and h["epoch"] == r["epoch"]
    assert h["num_evals"] == len(r["history"])
    assert np.abs(A - A_ref).max() <= tol * max(1.0, np.abs(A_ref).max())
    if not kernel:
        assert np.abs(W - W_ref).max() <= tol * max(1.0, np.abs(W_ref).max()) * d
    for i, f in enumerate(("primal", "dual")):
        assert abs(h["history"][-1][f] - r["history"][-1][i]) <= 10 * tol * max(1.0, abs(r["history"][-1][i]))


def test_stopping_paths(ref, hostsim):
    K, labels = kernel_problem(n=60, dim=4, m=4, seed=3)
    # evaluation before the first epoch, epoch limit reached, and no evaluation until the end
    check_fit(ref, hostsim, "l2_topk_hinge", K, labels, True, np.float64, 1e-9, m=4,
              eval_on_start=True, max_epoch=2, epsilon=1e-9)
    check_fit(ref, hostsim, "l2_topk_hinge", K, labels, True, np.float64, 1e-9, m=4,
              eval_epoch=0, max_epoch=4)
    check_fit(ref, hostsim, "l2_topk_hinge", K, labels, True, np.float64, 1e-9, m=4,
              max_epoch=0)


def golden_check(case, result, A, W):
    from oracle.refapi import OBJECTIVES  # noqa: F401  (names only)
    f64 = case["data"].dtype == np.float64
    tol = 1e-9 if f64 else 2e-4
    assert result["status_code"] == case["status"]
    assert result["epoch"] == case["epoch"]
    assert result["num_evals"] == len(case["history"])
    assert np.abs(A - case["A"]).max() <= tol * max(1.0, np.abs(case["A"]).max())
    if not case["kernel"]:
        d = case["data"].shape[1]
        assert np.abs(W - case["W"]).max() <= tol * max(1.0, np.abs(case["W"]).max()) * d
    for rec, ref_rec in zip(result["history"], case["history"]):
        for i, f in enumerate(("primal", "dual")):
            assert abs(rec[f] - ref_rec[i]) <= 10 * tol * max(1.0, abs(ref_rec[i]))


def test_golden_fits(hostsim):
    from oracle.refapi import OBJECTIVES as IDS
    from tests.golden_util import fit_cases
    count = 0
    for c in fit_cases():
        A = np.zeros_like(c["A"]); W = np.zeros_like(c["W"])
        r = hostsim.fit(IDS[c["objective"]], c["data"], c["labels"], A, W=None if c["kernel"] else W,
                        kernel=c["kernel"], c=c["c"], gamma=c["gamma"], k=c["k"], epsilon=c["epsilon"],
                        max_epoch=c["max_epoch"], eval_epoch=c["eval_epoch"], offsets=c["offsets"])
        golden_check(c, r, A, W)
        count += 1
    assert count == 36


def test_golden_epoch_orders(hostsim):
    from tests.golden_util import epoch_orders
    big, small = epoch_orders()
    assert np.array_equal(hostsim.epoch_permutations(50000, 2)[:, :64], big)
    assert np.array_equal(hostsim.epoch_permutations(1000, 3), small)
