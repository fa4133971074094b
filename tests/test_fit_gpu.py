"""Parity of the device fit (one launch per SDCA step, evaluation per epoch;
through the C ABI) with the reference's solver::solve on the same problems:
status, epoch count, final dual / primal variables and the evaluation records."""
import numpy as np
import pytest

from libsdca_b200.synth import kernel_problem
from tests.test_oracle_restatement import random_problem
from tests.util import stable_seed

pytestmark = pytest.mark.gpu

HINGE = ("l2_hinge_topk", "l2_hinge_topk_smooth", "l2_topk_hinge", "l2_topk_hinge_smooth",
         "l2_entropy_topk", "l2_entropy")
REF_STATUS = ("none", "solving", "solved", "no_progress", "max_epoch", "max_cpu_time",
              "max_wall_time", "failed")


def dev(x):
    import torch
    return None if x is None else torch.from_numpy(np.ascontiguousarray(x)).cuda()


def run_both(ref, mod, objective, data, labels, m, kernel, dtype, permutations=None, **kw):
    from oracle.refapi import OBJECTIVES as IDS
    n, d = data.shape
    fit_kw = dict(epsilon=kw.pop("epsilon", 1e-3), max_epoch=kw.pop("max_epoch", 30),
                  eval_epoch=kw.pop("eval_epoch", 1), eval_on_start=kw.pop("eval_on_start", False))
    recompute = kw.pop("recompute_primal", False)   # the reference's build here is the default one
    A_ref = np.zeros((n, m), dtype=dtype); W_ref = np.zeros((m, d), dtype=dtype)
    r = ref.fit(objective, data, A_ref, labels, W=None if kernel else W_ref, kernel=kernel,
                **fit_kw, **kw)
    A = dev(np.zeros((n, m), dtype=dtype)); W = None if kernel else dev(np.zeros((m, d), dtype=dtype))
    g = mod.fit_(IDS[objective], dev(data), dev(labels), A, W=W, kernel=kernel,
                 permutations=permutations, recompute_primal=recompute, **fit_kw, **kw)
    return r, g, A_ref, W_ref, A.cpu().numpy(), None if kernel else W.cpu().numpy()


def compare(r, g, A_ref, W_ref, A, W, tol, what):
    assert g["status"] == REF_STATUS[r["status"]], (what, g["status"], r["status"])
    assert g["epoch"] == r["epoch"], what
    assert g["num_evals"] == len(r["history"]), what
    # final variables: |difference| against the largest variable
    assert np.abs(A - A_ref).max() <= tol * max(1.0, np.abs(A_ref).max()), (what, np.abs(A - A_ref).max())
    if W is not None:
        assert np.abs(W - W_ref).max() <= tol * max(1.0, np.abs(W_ref).max()) * W.shape[1], what
    for e, (rec, ref_rec) in enumerate(zip(g["history"], r["history"])):
        for i, f in enumerate(("primal", "dual")):
            assert abs(rec[f] - ref_rec[i]) <= 10 * tol * max(1.0, abs(ref_rec[i])), (what, e, f)


@pytest.mark.parametrize("objective", HINGE)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_kernel_fit_matches_reference(ref, cuda_lib, objective, dtype):
    tol = 1e-9 if dtype == np.float64 else 2e-4
    for n, dim, m, k in ((120, 8, 6, 1), (700, 16, 37, 3), (1500, 32, 150, 5)):
        K, labels = kernel_problem(n=n, dim=dim, m=m, seed=stable_seed("gpu-fit", objective, n) % 1000,
                                   dtype=dtype)
        out = run_both(ref, cuda_lib, objective, K, labels, m, True, dtype, c=1.0, gamma=0.5, k=k,
                       max_epoch=15)
        compare(*out, tol, (objective, n, m, k))


@pytest.mark.parametrize("objective", HINGE)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_feature_fit_matches_reference(ref, cuda_lib, objective, dtype):
    rng = np.random.default_rng(stable_seed("gpu-fit-features", objective, str(dtype)))
    tol = 1e-9 if dtype == np.float64 else 2e-4
    for n, d, m, k in ((90, 7, 5, 2), (600, 50, 40, 1), (400, 300, 20, 4)):
        X, labels, _ = random_problem(rng, n, d, m, dtype, False)
        out = run_both(ref, cuda_lib, objective, X, labels, m, False, dtype, c=0.7, gamma=1.0, k=k,
                       max_epoch=10, eval_epoch=2)
        compare(*out, tol, (objective, n, d, m, k))


@pytest.mark.parametrize("objective", ["l2_multilabel_hinge", "l2_multilabel_hinge_smooth",
                                       "l2_multilabel_entropy"])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("kernel", [False, True])
def test_multilabel_fit_matches_reference(ref, cuda_lib, objective, dtype, kernel):
    from oracle.refapi import OBJECTIVES as IDS
    rng = np.random.default_rng(stable_seed("gpu-fit-multilabel", objective, str(dtype), kernel))
    tol = 1e-9 if dtype == np.float64 else 2e-4
    for n, d, m in ((70, 6, 7), (500, 40, 45)):
        X, labels, offsets = random_problem(rng, n, d, m, dtype, True)
        data = (X.astype(np.float64) @ X.astype(np.float64).T).astype(dtype) if kernel else X
        kw = dict(c=0.9, gamma=0.7, k=1, epsilon=1e-3, max_epoch=12, eval_epoch=2)
        A_ref = np.zeros((n, m), dtype=dtype); W_ref = np.zeros((m, d), dtype=dtype)
        r = ref.fit(objective, data, A_ref, labels, W=None if kernel else W_ref, kernel=kernel,
                    offsets=offsets, **kw)
        A = dev(np.zeros((n, m), dtype=dtype)); W = None if kernel else dev(np.zeros((m, d), dtype=dtype))
        g = cuda_lib.fit_(IDS[objective], dev(data), dev(labels), A, W=W, kernel=kernel,
                          offsets=dev(offsets), **kw)
        compare(r, g, A_ref, W_ref, A.cpu().numpy(), None if kernel else W.cpu().numpy(), tol,
                (objective, n, m, kernel))


def test_crammer_singer_medium(ref, cuda_lib):
    """The shape of the full-size problem at a size the CPU solver finishes quickly:
    RBF kernel of Gaussian blobs, msvm (top-k hinge beta, k = 1), gap checked every epoch."""
    K, labels = kernel_problem(n=4000, dim=128, m=100, seed=11)
    out = run_both(ref, cuda_lib, "l2_topk_hinge", K, labels, 100, True, np.float64, c=1.0, k=1,
                   max_epoch=50)
    compare(*out, 1e-9, "crammer-singer n=4000")
    assert out[1]["status"] == "solved"


def test_stopping_paths_and_given_order(ref, cuda_lib):
    K, labels = kernel_problem(n=200, dim=4, m=4, seed=3)
    args = (ref, cuda_lib, "l2_topk_hinge", K, labels, 4, True, np.float64)
    compare(*run_both(*args, eval_on_start=True, max_epoch=2, epsilon=1e-9), 1e-9, "on start")
    compare(*run_both(*args, eval_epoch=0, max_epoch=4), 1e-9, "no evaluation until the end")
    compare(*run_both(*args, max_epoch=0), 1e-9, "no epochs")
    # an order passed in by the caller is followed as given
    perm = cuda_lib.epoch_permutations(200, 6)
    assert np.array_equal(perm, ref.epoch_permutations(200, 6))
    compare(*run_both(*args, max_epoch=6, epsilon=0.0, permutations=perm), 1e-9, "given order")


def test_float_thresholds_reach_the_same_solution(cuda_lib):
    """opts.precision = 'single' of the reference's front end: thresholds and sums of
    the step in float.  The reference's compiled solver here is double only, so the
    check is against the double run: same objective values to float accuracy."""
    K, labels = kernel_problem(n=900, dim=16, m=30, seed=5)
    runs = {}
    for precision in ("double", "float"):
        A = dev(np.zeros((900, 30)))
        runs[precision] = cuda_lib.fit_(4, dev(K), dev(labels), A, kernel=True, c=1.0, k=1,
                                        precision=precision, max_epoch=40, eval_epoch=1)
        assert runs[precision]["status"] == "solved"
    d, f = runs["double"]["history"][-1], runs["float"]["history"][-1]
    assert abs(d["dual"] - f["dual"]) <= 2e-3 * abs(d["dual"])
    assert abs(d["primal"] - f["primal"]) <= 2e-3 * abs(d["primal"])


def test_many_classes_take_the_general_step(ref, cuda_lib):
    """More than 256 classes: the step runs the general threshold routines."""
    K, labels = kernel_problem(n=400, dim=16, m=300, seed=9)
    out = run_both(ref, cuda_lib, "l2_topk_hinge", K, labels, 300, True, np.float64, c=1.0, k=2,
                   max_epoch=4)
    compare(*out, 1e-9, "m=300")


def test_score_rows_that_do_not_fit_on_chip(ref, cuda_lib):
    """600 classes: the 64 score rows of a block (64 x 600 doubles) stay in global memory."""
    K, labels = kernel_problem(n=260, dim=16, m=600, seed=13)
    out = run_both(ref, cuda_lib, "l2_hinge_topk", K, labels, 600, True, np.float64, c=1.0, k=3,
                   max_epoch=3)
    compare(*out, 1e-9, "m=600")
    rng = np.random.default_rng(77)
    X, labels, _ = random_problem(rng, 150, 20, 600, np.float32, False)
    out = run_both(ref, cuda_lib, "l2_topk_hinge", X, labels, 600, False, np.float32, c=1.0, k=2,
                   max_epoch=3)
    compare(*out, 2e-4, "m=600 features")


def test_rejects_what_it_cannot_fit(cuda_lib):
    from libsdca_b200.binding import SdcabError
    K, labels = kernel_problem(n=50, dim=4, m=4, seed=3)
    A = dev(np.zeros((50, 4)))
    with pytest.raises(SdcabError):
        cuda_lib.fit_(6, dev(K), dev(labels), A, kernel=True)   # multilabel objective without offsets
    with pytest.raises(SdcabError):
        cuda_lib.fit_(4, dev(K[:, :40].copy()), dev(labels), A, kernel=True)  # kernel not square


def test_golden_fits(cuda_lib):
    """The committed fits of the reference's solver, without the reference at hand."""
    from oracle.refapi import OBJECTIVES as IDS
    from tests.golden_util import epoch_orders, fit_cases
    from tests.test_hostsim_fit import golden_check
    for c in fit_cases():
        A = dev(np.zeros_like(c["A"])); W = None if c["kernel"] else dev(np.zeros_like(c["W"]))
        r = cuda_lib.fit_(IDS[c["objective"]], dev(c["data"]), dev(c["labels"]), A, W=W,
                          kernel=c["kernel"], c=c["c"], gamma=c["gamma"], k=c["k"],
                          epsilon=c["epsilon"], max_epoch=c["max_epoch"], eval_epoch=c["eval_epoch"],
                          offsets=dev(c["offsets"]))
        golden_check(c, r, A.cpu().numpy(), None if c["kernel"] else W.cpu().numpy())
    big, small = epoch_orders()
    assert np.array_equal(cuda_lib.epoch_permutations(50000, 2)[:, :64], big)
    assert np.array_equal(cuda_lib.epoch_permutations(1000, 3), small)


def test_host_buffer_fit(ref, cuda_lib):
    """sdcab_fit_f64 / _f32: numpy in, numpy out, copies inside."""
    from libsdca_b200.binding import SdcabError
    for dtype, tol in ((np.float64, 1e-9), (np.float32, 2e-4)):
        K, labels = kernel_problem(n=300, dim=8, m=12, seed=21, dtype=dtype)
        A_ref = np.zeros((300, 12), dtype=dtype); A = np.zeros((300, 12), dtype=dtype)
        r = ref.fit("l2_topk_hinge", K, A_ref, labels, kernel=True, c=1.0, k=2, max_epoch=10, eval_epoch=1)
        g = cuda_lib.fit_(4, K, labels, A, kernel=True, c=1.0, k=2, max_epoch=10, eval_epoch=1)
        compare(r, g, A_ref, None, A, None, tol, "host buffers, kernel")
    rng = np.random.default_rng(5)
    X, labels, _ = random_problem(rng, 200, 9, 6, np.float64, False)
    A_ref = np.zeros((200, 6)); W_ref = np.zeros((6, 9)); A = np.zeros((200, 6)); W = np.zeros((6, 9))
    r = ref.fit("l2_entropy", X, A_ref, labels, W=W_ref, c=1.0, max_epoch=6, eval_epoch=2)
    g = cuda_lib.fit_(0, X, labels, A, W=W, c=1.0, max_epoch=6, eval_epoch=2)
    compare(r, g, A_ref, W_ref, A, W, 1e-9, "host buffers, features")
    bad = labels.copy(); bad[3] = 6
    with pytest.raises(SdcabError):
        cuda_lib.fit_(0, X, bad, A, W=W, c=1.0, max_epoch=1)


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_primal_from_dual_matches_matrix_product(cuda_lib, dtype):
    """W = [W0 +] X A' (eval_recompute_primal of the reference): ragged tiles, a
    launch that splits the examples into slices, with and without W0."""
    import torch
    rng = np.random.default_rng(stable_seed("primal-from-dual", str(dtype)))
    # the last three are shapes the tensor-core form takes for float data (2048 examples and
    # more, m and d multiples of four): ragged 256 x 256 tiles, more tiles than SM pairs'
    # first round, a contraction that is not a multiple of the stage
    for d, m, n in ((5, 3, 7), (128, 100, 1000), (300, 70, 4097), (4100, 10, 33), (1, 1, 1),
                    (256, 100, 5000), (520, 1000, 3001), (4096, 12, 2048)):
        X = rng.standard_normal((n, d)).astype(dtype)
        A = rng.standard_normal((n, m)).astype(dtype)
        W0 = rng.standard_normal((m, d)).astype(dtype)
        exact = A.astype(np.float64).T @ X.astype(np.float64)
        scale = np.abs(A.astype(np.float64)).T @ np.abs(X.astype(np.float64)) + 1.0
        tol = 1e-13 if dtype == np.float64 else 2e-6
        W = cuda_lib.primal_from_dual(dev(X), dev(A)).cpu().numpy()
        assert (np.abs(W - exact) <= tol * np.sqrt(n) * scale).all(), (d, m, n)
        W = cuda_lib.primal_from_dual(dev(X), dev(A), W0=dev(W0)).cpu().numpy()
        assert (np.abs(W - (exact + W0)) <= tol * np.sqrt(n) * (scale + np.abs(W0))).all(), (d, m, n, "W0")
        # the same call twice gives the same bits (fixed summation order)
        again = cuda_lib.primal_from_dual(dev(X), dev(A), W0=dev(W0)).cpu().numpy()
        assert np.array_equal(W, again)
        if dtype == np.float32 and n >= 2048 and m % 4 == 0 and d % 4 == 0:
            # the CUDA-core kernel (test switch) is a different kernel with the same answer
            from libsdca_b200 import binding as b
            try:
                b.test_set("primal_simt", 1)
                simt = cuda_lib.primal_from_dual(dev(X), dev(A), W0=dev(W0)).cpu().numpy()
            finally:
                b.test_set("primal_simt", 0)
            assert not np.array_equal(W, simt)
            assert (np.abs(W - simt) <= 2 * tol * np.sqrt(n) * (scale + np.abs(W0))).all(), (d, m, n, "simt")


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_feature_fit_with_recomputed_primal(ref, cuda_lib, dtype):
    """recompute_primal (the reference's SDCA_ACCURATE_MATH build rebuilds W from A
    before every evaluation): same fit within the tolerance of the default build, and
    the W it returns is X A' of the A it returns."""
    rng = np.random.default_rng(stable_seed("gpu-fit-recompute", str(dtype)))
    tol = 1e-9 if dtype == np.float64 else 2e-4
    for objective in ("l2_topk_hinge", "l2_entropy_topk"):
        X, labels, _ = random_problem(rng, 500, 60, 30, dtype, False)
        out = run_both(ref, cuda_lib, objective, X, labels, 30, False, dtype, c=0.7, gamma=1.0, k=2,
                       max_epoch=8, eval_epoch=2, recompute_primal=True)
        compare(*out, tol, (objective, "recompute"))
        A, W = out[4], out[5]
        exact = A.astype(np.float64).T @ X.astype(np.float64)
        wtol = 1e-12 if dtype == np.float64 else 1e-5
        assert np.abs(W - exact).max() <= wtol * max(1.0, np.abs(exact).max()) * 30
