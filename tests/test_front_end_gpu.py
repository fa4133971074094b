"""The callers either side of the fit, against the reference's solver: held-out sets
evaluated with every evaluation of the training set, test kernels K_tst = X_trn' X_tst, the
reference's own four-stage chain (features -> kernel warm start -> restart around W0 ->
kernel from scratch, test/solver/solver.cpp:93-126), and the matsdca_fit-like front end
(options in, model out, 0- or 1-based labels)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def blobs(rng, n, d, m, sep=2.5, dtype=np.float64):
    means = rng.standard_normal((m, d)) * sep
    labels = rng.integers(0, m, n).astype(np.int64)
    labels[:m] = np.arange(m)
    X = (means[labels] + rng.standard_normal((n, d))).astype(dtype)
    return X, labels, means


def test_held_out_sets_are_evaluated_with_every_evaluation(ref, cuda_lib):
    rng = np.random.default_rng(41)
    n, d, m = 600, 12, 7
    X, labels, means = blobs(rng, n, d, m)
    # small features: on well separated blobs of unit scale the reference's top-k entropy
    # steps saturate (arguments of order -1000) and its solver ends with no_progress along a
    # path that the last bits of the scores decide; at this scale every objective converges
    X *= 0.1
    sets = []
    for nt in (150, 90):
        lt = rng.integers(0, m, nt).astype(np.int64)
        sets.append((0.1 * (means[lt] + 1.3 * rng.standard_normal((nt, d))), lt))
    for objective, kw in (("l2_topk_hinge", dict(c=1.0, k=2)), ("l2_entropy_topk", dict(c=0.1, k=2)),
                          ("l2_hinge_topk_smooth", dict(c=1.0, k=2, gamma=0.7))):
        for kernel in (False, True):
            if kernel:
                data = np.ascontiguousarray(X @ X.T)
                tests = [(np.ascontiguousarray(t @ X.T), l) for t, l in sets]     # columns X_trn' x_tst
            else:
                data, tests = X, sets
            A_ref = np.zeros((n, m)); W_ref = np.zeros((m, d))
            r = ref.fit(objective, data, A_ref, labels, W=None if kernel else W_ref, kernel=kernel,
                        max_epoch=30, eval_epoch=3, tests=tests, **kw)
            A = np.zeros((n, m)); W = np.zeros((m, d))
            # matsdca_fit's names: gamma > 0 selects the smoothed class (mex_solve.cpp:660-675)
            g = cuda_lib.fit_(objective.replace("_smooth", ""), data, labels, A, W=None if kernel else W, kernel=kernel,
                              max_epoch=30, eval_epoch=3, tests=tests, gamma=kw.get("gamma", 0.0),
                              c=kw["c"], k=kw["k"])
            what = (objective, kernel)
            assert g["status_code"] == r["status"] and g["epoch"] == r["epoch"], what
            assert g["num_evals"] == len(r["history"]), what
            assert np.array_equal(g["eval_epoch"], r["history"][:, 7].astype(np.int64)), what
            for i, rec in enumerate(g["history"]):
                for j, f in enumerate(("primal", "dual")):
                    assert abs(rec[f] - r["history"][i][j]) <= 1e-9 * max(1, abs(r["history"][i][j])), what
            assert np.abs(A - A_ref).max() <= 1e-9 * max(1, np.abs(A_ref).max()), what
            for t in range(len(tests)):
                gt, rt = g["tests"][t], r["tests"][t]
                assert np.allclose(gt["primal_loss"], rt["primal_loss"], rtol=1e-9, atol=1e-12), what
                assert np.abs(gt["accuracy"] - rt["accuracy"]).max() <= 1e-12, what
            # the training accuracies of the last evaluation are the reference's
            assert np.abs(g["train_accuracy"][-1] - r["accuracy"]).max() <= 1e-12, what


def test_test_kernel_from_features_is_the_scores_product(cuda_lib):
    """K_tst = X_trn' X_tst (mex_solve.cpp:96-100) is the batched score product with the
    training examples in the place of the classes."""
    import torch
    from tests.test_scores_gpu import scores
    rng = np.random.default_rng(3)
    Xtrn = rng.standard_normal((333, 40)); Xtst = rng.standard_normal((77, 40))
    K = scores(cuda_lib, Xtst, W=Xtrn)          # (n_tst, n_trn): column i of K_tst per row
    assert np.abs(K - Xtst @ Xtrn.T).max() <= 1e-12 * 40


def test_reference_chain_features_kernel_prox_restart(ref, cuda_lib):
    """test/solver/solver.cpp:93-126: fit on features; warm-start the kernel problem from
    those dual variables (solved at once); restart around W0 = W with A = 0; kernel from
    scratch.  Every stage must reproduce the reference's status, epochs and objectives."""
    rng = np.random.default_rng(17)
    n, d, m = 300, 6, 5
    X, labels, _ = blobs(rng, n, d, m, sep=3.0)
    K = np.ascontiguousarray(X @ X.T)
    kw = dict(c=1.0, gamma=1.0, k=1)
    obj = "l2_topk_hinge_smooth"      # the reference's class; matsdca_fit's name is msvm_smooth
    name = "msvm_smooth"

    def compare(g, r, what):
        assert g["status_code"] == r["status"] and g["epoch"] == r["epoch"], what
        assert len(g["history"]) == len(r["history"]), what
        for i, rec in enumerate(g["history"]):
            for j, f in enumerate(("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer",
                                   "dual_regularizer")):
                assert abs(rec[f] - r["history"][i][j]) <= 1e-9 * max(1, abs(r["history"][i][j])), (what, i, f)

    # 1. features
    A_ref = np.zeros((n, m)); W_ref = np.zeros((m, d))
    r1 = ref.fit(obj, X, A_ref, labels, W=W_ref, **kw)
    A = np.zeros((n, m)); W = np.zeros((m, d))
    g1 = cuda_lib.fit_(name, X, labels, A, W=W, **kw)
    compare(g1, r1, "features")
    assert r1["status"] == 2      # solved
    # 2. kernel, warm start from the same dual variables, evaluated on start
    r2 = ref.fit(obj, K, A_ref, labels, kernel=True, eval_on_start=True, **kw)
    g2 = cuda_lib.fit_(name, K, labels, A, kernel=True, eval_on_start=True, **kw)
    compare(g2, r2, "kernel warm start")
    assert r2["epoch"] <= 10
    # 3. restart around W0: A = 0, W = W0 before the first step
    W0_ref = W_ref.copy(); W0 = W.copy()
    A_ref[:] = 0; A[:] = 0
    r3 = ref.fit(obj, X, A_ref, labels, W=W_ref, W0=W0_ref, eval_on_start=True, **kw)
    g3 = cuda_lib.fit_(name, X, labels, A, W=W, W0=W0, eval_on_start=True, **kw)
    compare(g3, r3, "prox restart")
    assert np.abs(W - W_ref).max() <= 1e-9 * max(1, np.abs(W_ref).max())
    # 4. kernel from scratch
    A_ref[:] = 0; A[:] = 0
    r4 = ref.fit(obj, K, A_ref, labels, kernel=True, eval_on_start=True, **kw)
    g4 = cuda_lib.fit_(name, K, labels, A, kernel=True, eval_on_start=True, **kw)
    compare(g4, r4, "kernel from scratch")
    assert r4["epoch"] > 0
    assert np.abs(A - A_ref).max() <= 1e-9 * max(1, np.abs(A_ref).max())


def test_train_front_end(ref, cuda_lib):
    """Options in, model out: the reference's defaults (msvm_smooth, c = gamma = k = 1,
    epsilon 1e-3, eval_epoch 10), 1-based labels, a held-out set, a Gram-matrix run."""
    rng = np.random.default_rng(23)
    n, d, m = 400, 8, 6
    X, labels, means = blobs(rng, n, d, m)
    lt = rng.integers(0, m, 120).astype(np.int64)
    Xt = means[lt] + 1.2 * rng.standard_normal((120, d))
    model = cuda_lib.train([X, Xt], [labels + 1, lt + 1])          # Matlab-style labels
    A_ref = np.zeros((n, m)); W_ref = np.zeros((m, d))
    r = ref.fit("l2_topk_hinge_smooth", X, A_ref, labels, W=W_ref, c=1.0, gamma=1.0, k=1,
                epsilon=1e-3, max_epoch=1000, eval_epoch=10, tests=[(Xt, lt)])
    assert model["objective"] == "msvm_smooth" and model["labels_one_based"]
    assert (model["num_dimensions"], model["num_examples"], model["num_classes"]) == (d, n, m)
    assert model["status"] == "solved" and r["status"] == 2 and model["epoch"] == r["epoch"]
    assert model["num_evals"] == len(r["history"])
    assert np.abs(model["A"] - A_ref).max() <= 1e-9 and np.abs(model["W"] - W_ref).max() <= 1e-9
    last = r["history"][-1]
    gap = (last[0] - last[1]) / max(abs(last[0]), abs(last[1]))
    assert abs(model["relative_gap"] - gap) <= 1e-9
    assert np.abs(model["tests"][0]["accuracy"] - r["tests"][0]["accuracy"]).max() <= 1e-12
    assert np.allclose(model["tests"][0]["primal_loss"], r["tests"][0]["primal_loss"], rtol=1e-9)
    # Gram matrices, float32, another objective
    K = np.ascontiguousarray((X @ X.T).astype(np.float32))
    Kt = np.ascontiguousarray((Xt @ X.T).astype(np.float32))
    model = cuda_lib.train([K, Kt], [labels, lt], objective="topk_hinge_beta", c=2.0, gamma=0.0, k=2,
                           is_dual=True, max_epoch=40, eval_epoch=4)
    A_ref = np.zeros((n, m), dtype=np.float32)
    r = ref.fit("l2_topk_hinge", K, A_ref, labels, kernel=True, c=2.0, k=2, max_epoch=40, eval_epoch=4,
                tests=[(Kt, lt)])
    assert model["is_dual"] and model["W"] is None
    assert model["epoch"] == r["epoch"] and model["num_evals"] == len(r["history"])
    assert np.abs(model["A"] - A_ref).max() <= 2e-4 * max(1, np.abs(A_ref).max())
    assert np.abs(model["tests"][0]["accuracy"] - r["tests"][0]["accuracy"]).max() <= 2.0 / 120
    # argument errors keep the reference's identifiers
    with pytest.raises(cuda_lib.SdcabError) as e:
        cuda_lib.train(X, labels + 2)
    assert e.value.status == -5
    with pytest.raises(cuda_lib.SdcabError) as e:
        cuda_lib.train(X, labels, objective="no_such_objective")
    assert e.value.status == -7
