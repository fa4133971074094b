"""Parity of the device evaluation (score GEMM + loss kernels, through the C ABI)
with the reference's evaluate_dataset, term by term."""
import os

import ctypes as C

import numpy as np
import pytest

from tests.golden_util import eval_cases
from tests.test_oracle_restatement import OBJECTIVES, random_problem
from tests.util import stable_seed

pytestmark = pytest.mark.gpu

FIELDS = ("primal", "dual", "primal_loss", "dual_loss", "primal_regularizer",
          "dual_regularizer", "rank_loss")


def compare(rec, ref_rec, tol, what="", reg_tol=None, acc_atol=1e-12):
    """Term-by-term comparison.  For float32 data the reference sums ||W||^2 (and
    <a_i, scores_i>) in float, in index order; that sum is only accurate to about
    count * FLT_EPSILON / 4, so the regulariser terms (and the totals that contain
    them) get that bound (reg_tol) while the loss terms keep the plain tolerance."""
    for f in FIELDS:
        t = tol
        if reg_tol is not None and ("regularizer" in f or f in ("primal", "dual")):
            t = max(tol, reg_tol)
        assert abs(rec[f] - ref_rec[f]) <= t * max(1, abs(ref_rec[f])), (what, f, rec[f], ref_rec[f])
    assert np.allclose(rec["accuracy"], ref_rec["accuracy"], atol=acc_atol), what


def float_sum_tol(dtype, count):
    return None if np.dtype(dtype) == np.float64 else count * float(np.finfo(np.float32).eps) / 4


def dev(x):
    import torch
    return None if x is None else torch.from_numpy(np.ascontiguousarray(x)).cuda()


def gpu_eval(mod, objective, X, labels, A=None, W=None, W0=None, offsets=None, device=True, **kw):
    from oracle.refapi import OBJECTIVES as IDS
    oid = IDS[objective]
    if device:
        return mod.evaluate(oid, dev(X), dev(labels), A=dev(A), W=dev(W), W0=dev(W0),
                            offsets=dev(offsets), **kw)
    return mod.evaluate(oid, X, labels, A=A, W=W, W0=W0, offsets=offsets, **kw)


@pytest.mark.parametrize("objective", OBJECTIVES)
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("kernel", [False, True])
def test_every_objective_matches_reference(ref, cuda_lib, objective, dtype, kernel):
    from oracle.refapi import MULTILABEL, OBJECTIVES as IDS
    rng = np.random.default_rng(stable_seed("gpu-eval", objective, str(dtype), kernel))
    ml = IDS[objective] in MULTILABEL
    for n, d, m, k in ((130, 12, 7, 2), (70, 37, 133, 5), (9, 3, 2, 1), (300, 64, 1000, 5)):
        if ml and m == 2:
            continue
        X, labels, offsets = random_problem(rng, n, d, m, dtype, ml)
        A = np.zeros((n, m), dtype=dtype); W = np.zeros((m, d), dtype=dtype)
        kw = dict(c=1.5, gamma=0.7, k=k)
        ref.fit(objective, X, A, labels, W=W, offsets=offsets, max_epoch=2, eval_epoch=10, **kw)
        tol = 1e-12 if dtype == np.float64 else 1e-5
        if kernel:
            K = (X.astype(np.float64) @ X.astype(np.float64).T).astype(dtype)
            r = ref.evaluate(objective, K, A.copy(), labels, kernel=True, offsets=offsets, **kw)
            g = gpu_eval(cuda_lib, objective, K, labels, A=A, offsets=offsets, kernel=True, **kw)
            h = gpu_eval(cuda_lib, objective, K, labels, A=A, offsets=offsets, kernel=True,
                         device=False, **kw)
        else:
            r = ref.evaluate(objective, X, A.copy(), labels, W=W, offsets=offsets, **kw)
            g = gpu_eval(cuda_lib, objective, X, labels, A=A, W=W, offsets=offsets, **kw)
            h = gpu_eval(cuda_lib, objective, X, labels, A=A, W=W, offsets=offsets, device=False, **kw)
        reg_tol = float_sum_tol(dtype, m * (n if kernel else d))
        compare(g, r, tol, (objective, n, d, m, "device"), reg_tol)
        compare(h, r, tol, (objective, n, d, m, "host"), reg_tol)
        if not kernel:
            # the regulariser itself is exact: 0.5 ||W||^2 accumulated in double
            exact = 0.5 * float((W.astype(np.float64) ** 2).sum())
            assert abs(g["primal_regularizer"] - exact) <= 1e-12 * max(1, exact)


def test_golden_eval_records(cuda_lib):
    from oracle.refapi import EVAL_FIELDS
    for c in eval_cases():
        kw = dict(c=c["c"], gamma=c["gamma"], k=c["k"], offsets=c["offsets"])
        if c["kernel"]:
            g = gpu_eval(cuda_lib, c["objective"], c["data"], c["labels"], A=c["A"], kernel=True, **kw)
        else:
            g = gpu_eval(cuda_lib, c["objective"], c["data"], c["labels"], A=c["A"], W=c["W"], **kw)
        tol = 1e-12 if c["data"].dtype == np.float64 else 1e-5
        ref_rec = {f: c["record"][i] for i, f in enumerate(EVAL_FIELDS)}
        ref_rec["accuracy"] = c["accuracy"]
        compare(g, ref_rec, tol, c["objective"])


def test_held_out_set_and_prox_regularizer(ref, cuda_lib):
    rng = np.random.default_rng(4)
    n, d, m = 90, 20, 11
    X, labels, _ = random_problem(rng, n, d, m, np.float64, False)
    A = np.zeros((n, m)); W = np.zeros((m, d))
    ref.fit("msvm_smooth", X, A, labels, W=W, max_epoch=2, eval_epoch=10, c=1.0, gamma=1.0, k=1)
    W0 = rng.standard_normal((m, d)) * 0.1
    r = ref.evaluate("msvm_smooth", X, A.copy(), labels, W=W, W0=W0, c=1.0, gamma=1.0, k=1)
    g = gpu_eval(cuda_lib, "msvm_smooth", X, labels, A=A, W=W, W0=W0, c=1.0, gamma=1.0, k=1)
    compare(g, r, 1e-12, "W0")
    rt = ref.evaluate("msvm_smooth", X[:30], A, labels[:30], W=W, is_train=False, c=1.0, gamma=1.0, k=1)
    gt = gpu_eval(cuda_lib, "msvm_smooth", X[:30], labels[:30], W=W, A=None, is_train=False,
                  c=1.0, gamma=1.0, k=1)
    assert abs(rt["primal_loss"] - gt["primal_loss"]) <= 1e-12 * max(1, abs(rt["primal_loss"]))
    assert np.allclose(rt["accuracy"], gt["accuracy"], atol=1e-12)


def test_config4_gap_terms_reduced_n(ref, cuda_lib):
    """Config 4 at reduced N: top-k hinge alpha, k = 5, d = 4096, m = 1000, float32;
    every term of the record is compared separately (the regulariser dwarfs the losses)."""
    from libsdca_b200 import synth
    n = 1024
    X, A, W, labels = synth.gap_problem(
        n=n, d=4096, m=1000, k=5, c=1.0,
        project=lambda v, k, rhs: ref.prox("topk_simplex", v, k=k, rhs=rhs))
    for objective, gamma in (("l2_hinge_topk", 0.0), ("l2_hinge_topk_smooth", 1.0)):
        r = ref.evaluate(objective, X, A.copy(), labels, W=W, c=1.0, gamma=gamma, k=5)
        g = gpu_eval(cuda_lib, objective, X, labels, A=A, W=W, c=1.0, gamma=gamma, k=5)
        # the reference sums ||W||^2 over 4.1e6 float products in a float accumulator
        # (its value is off by about half a percent here); the regulariser is
        # therefore checked against the exact double sum, the reference only
        # bounds it, and the loss terms are compared at the plain tolerance
        compare(g, r, 1e-5, objective, float_sum_tol(np.float32, 4096 * 1000), acc_atol=2.0 / n)
        exact = 0.5 * float((W.astype(np.float64) ** 2).sum())
        assert abs(g["primal_regularizer"] - exact) <= 1e-12 * exact
        assert abs(g["dual_regularizer"] - exact) <= 1e-12 * exact
        assert abs(g["primal"] - (g["primal_loss"] + exact)) <= 1e-9 * exact
        assert abs(g["dual"] - (g["dual_loss"] - exact)) <= 1e-9 * exact
        for f in ("primal_loss", "dual_loss"):
            assert abs(g[f] - r[f]) <= 1e-5 * max(1, abs(r[f])), (objective, f, g[f], r[f])
        assert np.abs(g["accuracy"] - r["accuracy"]).max() <= 2.0 / n



def test_chunked_evaluation_is_the_same(ref, cuda_lib):
    """A forced chunk length (the library's test switch) runs the chunk loop on a small
    problem; device and host-buffer forms must both give the unchunked result."""
    import torch
    from libsdca_b200 import binding as b
    from tests.test_oracle_restatement import random_problem
    rng = np.random.default_rng(8)
    X, labels, _ = random_problem(rng, 700, 16, 9, np.float64, False)
    A = rng.standard_normal((700, 9)) * 0.01
    W = rng.standard_normal((9, 16))
    t = lambda a: torch.from_numpy(a).cuda()
    fields = ("primal", "dual", "primal_loss", "dual_loss")
    outs = []
    try:
        for chunk in (0, 128):
            b.test_set("eval_chunk", chunk)
            for args in ((t(X), t(labels), t(A), t(W)), (X, labels, A, W)):
                r = cuda_lib.evaluate(5, args[0], args[1], A=args[2], W=args[3], c=1.0, gamma=0.5, k=1)
                outs.append(np.array([r[f] for f in fields] + r["accuracy"][:3].tolist()))
    finally:
        b.test_set("eval_chunk", 0)
    for o in outs[1:]:
        assert np.allclose(outs[0], o, rtol=1e-13, atol=0)


def test_host_form_shards_with_row_offsets(ref, cuda_lib):
    """Two shards of a training set through the host-buffer entry point, the second with
    a_row_offset > 0 into the whole A: their sums give the unsharded record and the
    reference's."""
    from libsdca_b200 import binding as b
    from tests.test_oracle_restatement import random_problem
    rng = np.random.default_rng(18)
    n, d, m = 600, 24, 11
    for kernel in (False, True):
        X = rng.standard_normal((n, n if kernel else d))      # kernel input: n columns of K
        labels = rng.integers(0, m, n).astype(np.int64)
        A = -np.abs(rng.standard_normal((n, m))) * 0.01
        A[np.arange(n), labels] = 0.03
        W = None if kernel else rng.standard_normal((m, d))
        whole = cuda_lib.evaluate("l2_entropy_topk", X, labels, A=A, W=W, kernel=kernel, c=1.0, k=3)
        r = ref.evaluate("l2_entropy_topk", X, A, labels, W=W, kernel=kernel, c=1.0, k=3)
        for f in ("primal", "dual", "primal_loss", "dual_loss"):
            assert abs(whole[f] - r[f]) <= 1e-12 * max(1, abs(r[f])), (kernel, f)
        # the same evaluation as two shards: device sums of each shard's host call are not
        # exposed, so compare the record terms that add up over shards
        cut = 250
        obj = b.make_objective("l2_entropy_topk", c=1.0, k=3)
        parts = []
        for first, count in ((0, cut), (cut, n - cut)):
            prob = b.make_problem(np.ascontiguousarray(X[first:first + count]),
                                  np.ascontiguousarray(labels[first:first + count]), A=A, W=W,
                                  kernel=kernel, a_row_offset=first,
                                  include_primal_regularizer=(first == 0))
            prob.m = m
            rec = b.EvalRecord()
            acc = np.zeros(m)
            fn = cuda_lib.lib().sdcab_eval_f64
            rc = fn(C.byref(obj), C.byref(prob), C.byref(rec), acc.ctypes.data_as(C.c_void_p))
            assert rc == 0
            parts.append((rec.primal_loss, rec.dual_loss, rec.primal_regularizer, rec.dual_regularizer))
        sums = np.sum(np.array(parts), axis=0)
        want = (whole["primal_loss"], whole["dual_loss"], whole["primal_regularizer"],
                whole["dual_regularizer"])
        assert np.allclose(sums, want, rtol=1e-12, atol=1e-14), (kernel, sums, want)


def test_host_forms_reject_bad_labels(cuda_lib):
    """Label checks of the reference (data/output.h:169-215) happen on the host, before
    anything is launched."""
    rng = np.random.default_rng(4)
    n, d, m = 20, 5, 4
    X = rng.standard_normal((n, d)); W = rng.standard_normal((m, d)); A = np.zeros((n, m))
    labels = rng.integers(0, m, n).astype(np.int64)
    bad = labels.copy(); bad[7] = m
    with pytest.raises(cuda_lib.SdcabError) as e:
        cuda_lib.evaluate("msvm", X, bad, A=A, W=W)
    assert e.value.status == -5
    bad[7] = -1
    with pytest.raises(cuda_lib.SdcabError) as e:
        cuda_lib.evaluate("msvm", X, bad, A=A, W=W)
    assert e.value.status == -5
    # multilabel: duplicate / unsorted labels, empty example, first offset not zero
    offsets = np.arange(0, 2 * n + 1, 2).astype(np.int64)
    ml = np.tile(np.array([0, 2], dtype=np.int64), n)
    assert np.isfinite(cuda_lib.evaluate("mlsvm", X, ml, A=A, W=W, offsets=offsets)["primal"])
    for mutate in ("dup", "unsorted", "empty", "first"):
        l2, o2 = ml.copy(), offsets.copy()
        if mutate == "dup": l2[1] = 0
        if mutate == "unsorted": l2[0], l2[1] = 2, 0
        if mutate == "empty": o2[3] = o2[2]
        if mutate == "first": o2[0] = 1
        with pytest.raises(cuda_lib.SdcabError) as e:
            cuda_lib.evaluate("mlsvm", X, l2, A=A, W=W, offsets=o2)
        assert e.value.status == -5, mutate


@pytest.mark.parametrize("objective", ["l2_hinge_topk", "l2_topk_hinge", "l2_hinge_topk_smooth"])
def test_register_row_loss_kernel_matches_reference_and_general_kernel(ref, cuda_lib, objective):
    """Float features with 64 to 1024 classes in whole 16-byte vectors take the loss
    kernel that keeps the score row in registers.  It must agree with the reference term
    by term, and with the library's general loss kernel (test switch) to rounding; the two
    are different kernels, so at least one shape must differ in the last bits."""
    from libsdca_b200 import binding as b
    rng = np.random.default_rng(stable_seed("loss-rows", objective))
    differ = False
    try:
        for n, d, m, k, gamma in ((257, 32, 64, 1, 1.0), (130, 48, 100, 3, 0.3), (200, 40, 260, 8, 2.0),
                                  (300, 64, 1000, 5, 1.0), (90, 64, 1024, 5, 0.05), (64, 32, 516, 2, 10.0)):
            X, labels, _ = random_problem(rng, n, d, m, np.float32, False)
            A = np.zeros((n, m), dtype=np.float32); W = np.zeros((m, d), dtype=np.float32)
            kw = dict(c=1.5, gamma=gamma, k=k)
            ref.fit(objective, X, A, labels, W=W, max_epoch=2, eval_epoch=10, **kw)
            r = ref.evaluate(objective, X, A.copy(), labels, W=W, **kw)
            reg_tol = float_sum_tol(np.float32, m * d)
            for precision in ("double", "single"):
                b.test_set("loss_general", 0)
                g = gpu_eval(cuda_lib, objective, X, labels, A=A, W=W, precision=precision, **kw)
                b.test_set("loss_general", 1)
                q = gpu_eval(cuda_lib, objective, X, labels, A=A, W=W, precision=precision, **kw)
                tol = 1e-5 if precision == "double" else 1e-4
                compare(g, r, tol, (objective, n, d, m, precision, "register rows"), reg_tol)
                compare(g, q, 1e-9 if precision == "double" else 1e-4,
                        (objective, n, d, m, precision, "against the general kernel"))
                assert np.array_equal(g["accuracy"], q["accuracy"])
                differ = differ or g["primal_loss"] != q["primal_loss"] or g["dual_loss"] != q["dual_loss"]
    finally:
        b.test_set("loss_general", 0)
    if objective == "l2_hinge_topk_smooth":
        assert differ
