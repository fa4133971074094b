"""The five workloads at their full sizes, checked through properties that do not
need a reference run of that size: feasibility of every row, idempotence,
run-to-run bit equality, additivity of the evaluation over shards of examples,
weak duality and monotone dual progress of the fit -- plus a sample of rows
against the reference (or the committed restatement when the reference's compiled
headers are not present)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def checker():
    from oracle import refapi
    return refapi.reference() if refapi.have_reference() else refapi.restatement()


def sample_rows(t, count, seed):
    import torch
    g = torch.Generator(device="cpu").manual_seed(seed)
    idx = torch.randperm(t.shape[0], generator=g)[:count].to(t.device)
    return idx, t[idx].cpu().numpy()


def test_config1_simplex_65536_by_100_f64(cuda_lib):
    import torch
    from libsdca_b200 import synth
    a = torch.from_numpy(synth.simplex_rows()).cuda()
    x = cuda_lib.prox(a, "knapsack")
    assert x.shape == (65536, 100)
    assert float(x.min()) >= 0.0
    assert float((x.sum(dim=1) - 1).abs().max()) <= 1e-12
    # the projection of a point of the simplex is the point itself
    again = cuda_lib.prox(x, "knapsack")
    assert float((again - x).abs().max()) <= 1e-14
    # order is preserved: a_i >= a_j implies x_i >= x_j
    order = a.argsort(dim=1)
    assert bool((torch.gather(x, 1, order).diff(dim=1) >= 0).all())
    idx, rows = sample_rows(a, 2048, 1)
    ref = checker().prox("knapsack", rows)
    assert np.abs(x[idx].cpu().numpy() - ref).max() <= 1e-12 * max(1.0, np.abs(rows).max())


@pytest.mark.parametrize("name", ["topk_simplex", "topk_cone"])
def test_config2_topk_262144_by_1000_f32(cuda_lib, name):
    import torch
    from libsdca_b200 import synth
    k = 5
    a = torch.from_numpy(synth.topk_rows()).cuda()
    kw = dict(k=k, rhs=1.0) if name == "topk_simplex" else dict(k=k)
    x = cuda_lib.prox(a, name, **kw)
    assert x.shape == (262144, 1000)
    total = x.double().sum(dim=1)
    assert float(x.min()) >= 0.0
    # every entry is at most the k-th part of the row's sum (include/sdca/prox/topk_cone.h:135-160)
    assert float((x.double().max(dim=1).values - total / k).max()) <= 1e-6
    if name == "topk_simplex":
        assert float(total.max()) <= 1.0 + 1e-5
    # idempotence, and the same bits on a second run
    again = cuda_lib.prox(x, name, **kw)
    assert float((again - x).abs().max()) <= 2e-6
    assert torch.equal(cuda_lib.prox(a, name, **kw), x)
    idx, rows = sample_rows(a, 2048, 2)
    ref = checker().prox(name, rows, **kw)
    scale = np.maximum(1, np.abs(rows).max(axis=1, keepdims=True))
    assert (np.abs(x[idx].cpu().numpy().astype(np.float64) - ref) / scale).max() <= 1e-5


@pytest.mark.parametrize("name,kw", [("knapsack", dict(lo=0.0, hi=1.0, rhs=1.0)),
                                     ("knapsack_le", dict(lo=0.0, hi=1.0, rhs=1.0)),
                                     ("knapsack_le_biased", dict(lo=0.0, hi=1.0, rhs=1.0, rho=1.0)),
                                     ("topk_cone_biased", dict(k=5, rho=1.0)),
                                     ("two_simplex", dict(p=500, rhs=1.0))])
def test_operator_sweep_131072_by_1000_f32(cuda_lib, name, kw):
    """The operators of the sweep (bench config 6) at its size: feasibility of every row,
    idempotence where the operator is a Euclidean projection, run-to-run bit equality, and a
    sample of rows against the reference."""
    import torch
    from libsdca_b200 import synth
    a = torch.from_numpy(synth.topk_rows(rows=131072)).cuda()
    x = cuda_lib.prox(a, name, **kw)
    assert x.shape == a.shape and bool(torch.isfinite(x).all())
    assert float(x.min()) >= 0.0
    total = x.double().sum(dim=1)
    if name == "knapsack":
        assert float((total - 1).abs().max()) <= 1e-5 and float(x.max()) <= 1.0
    elif name.startswith("knapsack_le"):
        assert float(total.max()) <= 1.0 + 1e-5 and float(x.max()) <= 1.0
    elif name == "topk_cone_biased":
        assert float((x.double().max(dim=1).values - total / kw["k"]).max()) <= 1e-6
    elif name == "two_simplex":
        sa, sb = x[:, :500].double().sum(dim=1), x[:, 500:].double().sum(dim=1)
        assert float((sa - sb).abs().max()) <= 1e-5 and float(sa.max()) <= 1.0 + 1e-5
    if name in ("knapsack", "knapsack_le", "two_simplex"):
        again = cuda_lib.prox(x, name, **kw)
        assert float((again - x).abs().max()) <= 2e-6
    assert torch.equal(cuda_lib.prox(a, name, **kw), x)
    idx, rows = sample_rows(a, 2048, 6)
    ref = checker().prox(name, rows, **kw)
    scale = np.maximum(1, np.abs(rows).max(axis=1, keepdims=True))
    assert (np.abs(x[idx].cpu().numpy().astype(np.float64) - ref) / scale).max() <= 1e-5


@pytest.mark.parametrize("k", [1, 10])
def test_config3_topk_entropy_1048576_by_200_f32(cuda_lib, k):
    import torch
    from libsdca_b200 import synth
    a = torch.from_numpy(synth.entropy_rows()).cuda()
    x = cuda_lib.prox(a, "topk_entropy", k=k)
    total = x.double().sum(dim=1)
    assert float(x.min()) >= 0.0
    assert float(total.max()) <= 1.0 + 1e-5                # <1, x> = s <= 1 (topk_entropy.h:10-19)
    assert float(total.min()) > 0.5                        # the best class of N(0, 4) scores carries mass
    assert float((x.double().max(dim=1).values - total / k).max()) <= 1e-6
    idx, rows = sample_rows(a, 1024, 3)
    ref = checker().prox("topk_entropy", rows, k=k)
    assert np.abs(x[idx].cpu().numpy().astype(np.float64) - ref).max() <= 1e-5


def test_config3_lambert_w_exp_full_count(cuda_lib):
    import torch
    from libsdca_b200 import synth
    x = torch.from_numpy(synth.lambert_inputs()).cuda()
    w = x.clone()
    cuda_lib.lambert_w_exp_(w)
    # w exp(w) = exp(x)  <=>  w + log(w) = x for w > 0; checked in double on the float result
    wd = w.double()
    ok = wd > 1e-30
    resid = (wd[ok] + wd[ok].log() - x.double()[ok]).abs()
    assert float(resid.max()) <= 2e-5 * 31
    assert float(w.min()) >= 0.0
    assert bool((w[x.argsort()].diff() >= 0).all())          # monotone
    assert abs(float(w[0]) - np.exp(-30.0)) <= 1e-5 * np.exp(-30.0) and float(w[1]) > 26.0


def test_config4_gap_1048576_examples_is_additive_over_shards(cuda_lib):
    """Full size: d = 4096, m = 1000, N = 1 048 576 float32.  The sums of four shards
    add up to the sums of the whole, primal >= dual at a feasible dual point, and
    256 examples agree with the CPU checker term by term."""
    import torch
    from libsdca_b200 import binding as b
    d, m, k, c, n = 4096, 1000, 5, 1.0, 1048576
    gen = torch.Generator(device="cuda").manual_seed(5)
    means = torch.randn((m, d), generator=gen, device="cuda")
    labels = torch.randint(0, m, (n,), generator=gen, device="cuda")
    X = torch.empty((n, d), device="cuda")
    for i in range(0, n, 65536):
        X[i:i + 65536] = means[labels[i:i + 65536]] + 2.0 * torch.randn((65536, d), generator=gen, device="cuda")
    v = torch.randn((n, m - 1), generator=gen, device="cuda")
    cuda_lib.prox_(v, "topk_simplex", k=k, rhs=c)
    A = torch.zeros((n, m), device="cuda")
    cols = torch.arange(m - 1, device="cuda")[None, :] + (torch.arange(m - 1, device="cuda")[None, :] >= labels[:, None])
    A.scatter_(1, cols, -v)
    A[torch.arange(n, device="cuda"), labels] = torch.clamp(v.double().sum(dim=1), max=c).float()
    del v, cols
    W = torch.zeros((m, d), device="cuda")
    for i in range(0, n, 65536):
        W += A[i:i + 65536].T @ X[i:i + 65536]
    obj = b.make_objective("topk_hinge_alpha", c=c, gamma=0.0, k=k)
    whole = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    cuda_lib.eval_sums_(obj, b.make_problem(X, labels, A=A, W=W), whole, "f32")
    parts = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    q = n // 4
    for s in range(4):
        part = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
        prob = b.make_problem(X[s * q:(s + 1) * q], labels[s * q:(s + 1) * q], A=A, W=W,
                              a_row_offset=s * q, include_primal_regularizer=(s == 0))
        cuda_lib.eval_sums_(obj, prob, part, "f32")
        parts += part
    whole, parts = whole.cpu().numpy(), parts.cpu().numpy()
    assert np.abs(whole - parts).max() <= 1e-9 * np.abs(whole).max()
    assert whole[8:].sum() == n and parts[8:].sum() == n           # every example has a rank
    rec = cuda_lib.eval_finish(obj, m, whole)
    assert rec["primal"] >= rec["dual"] - 1e-9 * abs(rec["primal"])
    # a slice against the CPU checker
    sl = slice(1000, 1256)
    r = checker().evaluate("l2_hinge_topk", X[sl].cpu().numpy(), A[sl].cpu().numpy(), labels[sl].cpu().numpy(),
                           W=W.cpu().numpy(), c=c, k=k)
    small = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    cuda_lib.eval_sums_(obj, b.make_problem(X[sl].contiguous(), labels[sl].contiguous(), A=A[sl].contiguous(), W=W),
                        small, "f32")
    g = cuda_lib.eval_finish(obj, m, small.cpu().numpy())
    for f in ("primal_loss", "dual_loss"):
        assert abs(g[f] - r[f]) <= 1e-5 * max(1.0, abs(r[f])), (f, g[f], r[f])
    # At this dual point the margins are huge (W sums a million examples), so every primal
    # loss above is zero.  The same slice with the dual point scaled down, and W built from
    # the slice alone, has margins of order one, some of them violated: there the loss terms of
    # both the plain and the smoothed objective are compared with the CPU checker's.
    scale = 2.5e-5
    Xs, ls = X[sl].contiguous(), labels[sl].contiguous()
    As = (A[sl] * scale).contiguous()
    Ws = (As.T @ Xs).contiguous()
    for name, gamma in (("l2_hinge_topk", 0.0), ("l2_hinge_topk_smooth", 1.0)):
        o = b.make_objective("topk_hinge_alpha", c=c, gamma=gamma, k=k)
        r = checker().evaluate(name, Xs.cpu().numpy(), As.cpu().numpy(), ls.cpu().numpy(),
                               W=Ws.cpu().numpy(), c=c, gamma=gamma, k=k)
        assert r["primal_loss"] > 1.0, (name, r["primal_loss"])    # margins really are violated
        small.zero_()
        cuda_lib.eval_sums_(o, b.make_problem(Xs, ls, A=As, W=Ws), small, "f32")
        g = cuda_lib.eval_finish(o, m, small.cpu().numpy())
        for f in ("primal_loss", "dual_loss"):
            assert abs(g[f] - r[f]) <= 1e-5 * max(1.0, abs(r[f])), (name, f, g[f], r[f])
        assert np.abs(g["accuracy"] - r["accuracy"]).max() <= 2.0 / 256
    # the smoothed objective (gamma = 1, the default of matsdca_fit) at full size: additive
    # over shards, primal >= dual
    obj1 = b.make_objective("topk_hinge_alpha", c=c, gamma=1.0, k=k)
    whole1 = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    cuda_lib.eval_sums_(obj1, b.make_problem(X, labels, A=A, W=W), whole1, "f32")
    parts1 = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
    for s in range(4):
        part = torch.zeros(8 + m, dtype=torch.float64, device="cuda")
        prob = b.make_problem(X[s * q:(s + 1) * q], labels[s * q:(s + 1) * q], A=A, W=W,
                              a_row_offset=s * q, include_primal_regularizer=(s == 0))
        cuda_lib.eval_sums_(obj1, prob, part, "f32")
        parts1 += part
    whole1, parts1 = whole1.cpu().numpy(), parts1.cpu().numpy()
    assert np.abs(whole1 - parts1).max() <= 1e-9 * np.abs(whole1).max()
    rec1 = cuda_lib.eval_finish(obj1, m, whole1)
    assert rec1["primal"] >= rec1["dual"] - 1e-9 * abs(rec1["primal"])
    assert rec1["dual_loss"] < rec["dual_loss"]     # the smoothing term -gamma/(2c) sum a_j^2 is there


def test_config5_crammer_singer_fit_50000_f64(cuda_lib):
    """Full size: RBF kernel of 50 000 blobs, m = 100, msvm, epsilon = 1e-3."""
    import torch
    n, m, dim = 50000, 100, 128
    g = torch.Generator(device="cuda"); g.manual_seed(6)
    means = torch.randn(m, dim, generator=g, device="cuda", dtype=torch.float64)
    labels = torch.randint(0, m, (n,), generator=g, device="cuda")
    P = means[labels] + 1.5 * torch.randn(n, dim, generator=g, device="cuda", dtype=torch.float64)
    sq = (P * P).sum(1)
    K = P @ P.T
    K.mul_(-2).add_(sq[:, None]).add_(sq[None, :]).clamp_(min=0).div_(-dim).exp_()
    A = torch.zeros(n, m, device="cuda", dtype=torch.float64)
    r = cuda_lib.fit_(4, K, labels, A, kernel=True, c=1.0, k=1, max_epoch=100, eval_epoch=1, epsilon=1e-3)
    assert r["status"] == "solved" and r["epoch"] <= 20
    hist = r["history"]
    assert hist[-1]["primal"] - hist[-1]["dual"] <= 1e-3 * max(abs(hist[-1]["primal"]), abs(hist[-1]["dual"]))
    for before, after in zip(hist, hist[1:]):
        assert after["dual"] >= before["dual"] - 1e-9 * abs(before["dual"])      # SDCA ascends the dual
        assert after["primal"] >= after["dual"]
    # feasibility of the dual point (objective/l2_topk_hinge.h:64-68): the label's variable is the
    # negated sum of the others, which lie in [-c/k, 0]
    off = A.clone(); off[torch.arange(n, device="cuda"), labels] = 0
    assert float(off.max()) <= 0.0 and float(off.min()) >= -1.0 - 1e-12
    assert float((A.sum(dim=1)).abs().max()) <= 1e-12
    # the same order of examples as the reference's solver
    perm = cuda_lib.epoch_permutations(n, 1)
    assert sorted(perm[0].tolist()) == list(range(n))
