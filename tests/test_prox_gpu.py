"""Parity of the CUDA prox kernels (through the C ABI) with the reference."""
import numpy as np
import pytest

from tests.util import float_precision_ok, stable_seed, PROX_SINGLE, random_opts, regime, scaled_error, tolerance, thresholds_agree, two_simplex_sort_defined

pytestmark = pytest.mark.gpu


def run_dev(mod, name, a, **kw):
    import torch
    t = torch.from_numpy(a).cuda()
    mod.prox_(t, name, **kw)
    torch.cuda.synchronize()
    return t.cpu().numpy()


@pytest.mark.parametrize("name", PROX_SINGLE + ["two_simplex", "two_simplex_sort"])
@pytest.mark.parametrize("dtype,precision", [(np.float64, "double"), (np.float32, "double"),
                                              (np.float32, "float")])
def test_regimes_match_reference(ref, cuda_lib, name, dtype, precision):
    # two_simplex_sort (prox/two_simplex_sort.h:24-111 of the reference) solves the same
    # problem as two_simplex by sorting; here it is compared under its own name with the
    # reference's sort-based routine
    rng = np.random.default_rng(stable_seed(name, str(dtype), precision, 1))
    for kind in ("normal", "pos", "neg", "mixed", "ties"):
        for m in (1, 2, 3, 5, 31, 32, 33, 200, 1023, 1024, 1025):
            if name.startswith("two_simplex") and m < 2:
                continue
            n = 37 if m < 1000 else 9
            a = regime(rng, n, m, dtype, kind)
            kw = random_opts(rng, name, m)
            if name == "two_simplex_sort":
                a = a[two_simplex_sort_defined(ref, a, result=precision, **kw)]
                if len(a) == 0:
                    continue
            x_ref = ref.prox(name, a, result=precision, **kw)
            x = run_dev(cuda_lib, name, a, precision=precision, **kw)
            tol = tolerance(dtype, precision, m)
            if precision == "double":
                err = scaled_error(x, x_ref, a).max()
                assert err <= tol, (name, kind, m, kw, err)
            else:
                ok, err = float_precision_ok(x, x_ref, ref.prox(name, a, result="double", **kw), a, tol)
                assert ok, (name, kind, m, kw, err)


def test_config1_simplex_f64(ref, cuda_lib):
    from libsdca_b200 import synth
    a = synth.simplex_rows(rows=8192)
    x = run_dev(cuda_lib, "knapsack", a)
    x_ref = ref.prox("knapsack", a)
    assert scaled_error(x, x_ref, a).max() <= 1e-12
    assert np.abs(x.sum(axis=1) - 1).max() < 1e-12


@pytest.mark.parametrize("dtype,precision", [(np.float64, "double"), (np.float32, "double"),
                                              (np.float32, "float")])
def test_simplex_candidate_path_matches_reference(ref, cuda_lib, dtype, precision):
    """knapsack_eq with lo = 0: rows whose support lies among the few entries above
    max - rhs are solved on those candidates; rows with an entry at the upper bound,
    with more than 32 candidates or with ties take the general routine or must agree
    with it."""
    rng = np.random.default_rng(stable_seed("simplex-candidates", str(dtype), precision))
    for m in (8, 100, 200, 512):
        a = np.concatenate([regime(rng, 300, m, dtype, kind)
                            for kind in ("normal", "pos", "neg", "mixed", "ties")])
        for kw in (dict(lo=0.0, hi=1.0, rhs=1.0), dict(lo=0.0, hi=1e30, rhs=0.3),
                   dict(lo=0.0, hi=0.4, rhs=1.0), dict(lo=0.0, hi=3.0, rhs=5.0)):
            x = run_dev(cuda_lib, "knapsack_eq", a, precision=precision, **kw)
            x_ref = ref.prox("knapsack_eq", a, result=precision, **kw)
            tol = tolerance(dtype, precision, m)
            if precision == "double":
                err = scaled_error(x, x_ref, a).max()
                assert err <= tol, (m, kw, err)
                assert np.abs(x.sum(axis=1, dtype=np.float64) - kw["rhs"]).max() <= max(tol, 1e-6 if dtype == np.float32 else 0) * max(1.0, kw["rhs"]) * m
            else:
                ok, err = float_precision_ok(x, x_ref, ref.prox("knapsack_eq", a, result="double", **kw), a, tol)
                assert ok, (m, kw, err)


@pytest.mark.parametrize("dtype,precision", [(np.float64, "double"), (np.float32, "double"),
                                              (np.float32, "float")])
def test_knapsack_family_and_biased_cone_candidate_paths(ref, cuda_lib, dtype, precision):
    """Long rows of knapsack_eq / _le / _le_biased (cut from the largest lane maxima, the
    clipped-sum test, the t >= rho * rhs test) and of the biased top-k cone (lane u solving
    the size-u search on the sorted candidates) against the reference, on rows that take the
    candidate paths and on rows that must fall back (bunched values, ties, tiny rho); and
    two_simplex, whose first phase is the simplex projection of each block."""
    from libsdca_b200 import synth
    rng = np.random.default_rng(stable_seed("candidate-paths", str(dtype), precision))
    for m in (64, 200, 1000):
        a = np.concatenate([regime(rng, 200, m, dtype, kind)
                            for kind in ("normal", "pos", "neg", "mixed", "ties")] +
                           [synth.topk_rows(rows=600, m=m, seed=int(rng.integers(1 << 30))).astype(dtype),
                            (3 * synth.topk_rows(rows=200, m=m, seed=int(rng.integers(1 << 30)))).astype(dtype)])
        cases = [("knapsack_le", dict(lo=0.0, hi=1.0, rhs=1.0)), ("knapsack_le", dict(lo=0.0, hi=0.3, rhs=2.0)),
                 ("knapsack_le", dict(lo=0.0, hi=1.0, rhs=1e4)),
                 ("knapsack_le_biased", dict(lo=0.0, hi=1.0, rhs=1.0, rho=1.0)),
                 ("knapsack_le_biased", dict(lo=0.0, hi=1.0, rhs=1.0, rho=5.0)),
                 ("knapsack_le_biased", dict(lo=0.0, hi=0.5, rhs=3.0, rho=0.0)),
                 ("knapsack_eq", dict(lo=0.0, hi=1.0, rhs=1.0)), ("knapsack_eq", dict(lo=0.0, hi=10.0, rhs=4.0))]
        for k in (1, 3, 5, 8):
            for rho in (1e-6, 0.05, 1.0, 7.0):
                cases.append(("topk_cone_biased", dict(k=k, rho=rho)))
        for p_ in (1, m // 4, m // 2 + 1, m - 1):
            for rhs in (0.2, 1.0, 50.0):
                cases.append(("two_simplex", dict(p=p_, rhs=rhs)))
        cases.append(("two_simplex_sort", dict(p=m // 2, rhs=1.0)))
        cases.append(("two_simplex_sort", dict(p=m // 3, rhs=30.0)))
        for name, kw in cases:
            rows = a
            if name == "two_simplex_sort":
                # rows on which the reference's walk stays inside its arrays
                rows = a[two_simplex_sort_defined(ref, a, result=precision, **kw)]
            x = run_dev(cuda_lib, name, rows, precision=precision, **kw)
            x_ref = ref.prox(name, rows, result=precision, **kw)
            tol = tolerance(dtype, precision, m)
            if precision == "double":
                err = scaled_error(x, x_ref, rows).max()
                assert err <= tol, (name, m, kw, err)
            else:
                ok, err = float_precision_ok(x, x_ref, ref.prox(name, rows, result="double", **kw), rows, tol)
                assert ok, (name, m, kw, err)


@pytest.mark.parametrize("name,kw", [("topk_simplex", dict(k=5, rhs=1.0)), ("topk_cone", dict(k=5))])
@pytest.mark.parametrize("precision", ["double", "float"])
def test_config2_topk_f32_with_ties(ref, cuda_lib, name, kw, precision):
    import torch
    from libsdca_b200 import synth
    a = synth.topk_rows(rows=4096)
    x = run_dev(cuda_lib, name, a, precision=precision, **kw)
    x_ref = ref.prox(name, a, result=precision, **kw)
    tol = tolerance(np.float32, precision, 1000)
    assert scaled_error(x, x_ref, a).max() <= tol
    # identical index sets of the entries at the upper bound and in the middle
    thr = cuda_lib.thresholds(torch.from_numpy(a).cuda(), name, precision=precision, **kw)
    rt = ref.thresholds(name, a, result=precision, **kw)
    differ = thresholds_agree(thr, rt, x, x_ref, a, tol)
    if precision == "double":
        hi = x_ref.max(axis=1, keepdims=True)
        assert np.array_equal(x == x.max(axis=1, keepdims=True), x_ref == hi)
        assert np.array_equal(x > 0, x_ref > 0)
        assert differ <= len(a) // 8  # only rows with tied values (10 % of the rows) may


@pytest.mark.parametrize("name,kw", [("topk_entropy", dict(k=1)), ("topk_entropy", dict(k=10)),
                                     ("entropy", dict(hi=1.0, rhs=1.0)),
                                     ("entropy_norm", dict(hi=1.0, rhs=1.0)),
                                     ("topk_entropy_biased", dict(k=10, alpha=1.0))])
def test_config3_entropy_f32(ref, cuda_lib, name, kw):
    from libsdca_b200 import synth
    rows = 4096 if "biased" not in name and "norm" not in name else 512
    a = synth.entropy_rows(rows=rows)
    x = run_dev(cuda_lib, name, a, **kw)
    x_ref = ref.prox(name, a, **kw)
    assert scaled_error(x, x_ref, a).max() <= 1e-5


@pytest.mark.parametrize("name", ["entropy", "topk_entropy"])
@pytest.mark.parametrize("precision", ["double", "float"])
def test_grouped_entropic_rows_match_reference(ref, cuda_lib, name, precision):
    """Enough float rows for the kernel that batches the scalar work of the entropic
    projections over groups of rows (it wants a group for every resident warp).  All
    regimes are shuffled into one matrix, so that a group mixes rows of the closed
    forms with rows that are handed to the general routine."""
    rng = np.random.default_rng(stable_seed(name, precision, 7))
    for m in (36, 200, 400):
        # 40 013 rows: the last group of a block is a ragged one
        a = np.concatenate([regime(rng, 8000 + (13 if kind == "normal" else 0), m, np.float32, kind)
                            for kind in ("normal", "pos", "neg", "mixed", "ties")])
        rng.shuffle(a, axis=0)
        if name == "entropy":
            variants = [dict(hi=1.0, rhs=1.0), dict(hi=0.05, rhs=1.0), dict(hi=0.4, rhs=0.7)]
        else:
            variants = [dict(k=1), dict(k=3), dict(k=10), dict(k=min(30, m // 2))]
        for kw in variants:
            x = run_dev(cuda_lib, name, a, precision=precision, **kw)
            x_ref = ref.prox(name, a, result=precision, **kw)
            tol = tolerance(np.float32, precision, m)
            if precision == "double":
                err = scaled_error(x, x_ref, a).max()
                assert err <= tol, (name, m, kw, err)
            else:
                ok, err = float_precision_ok(x, x_ref, ref.prox(name, a, result="double", **kw), a, tol)
                assert ok, (name, m, kw, err)
            # in place and out of place agree bit for bit
            import torch
            src = torch.from_numpy(a).cuda()
            dst = torch.empty_like(src)
            cuda_lib.prox_to(src, dst, name, precision=precision, **kw)
            assert np.array_equal(dst.cpu().numpy(), x)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_config3_lambert(ref, cuda_lib, dtype):
    import torch
    from libsdca_b200 import synth
    x = synth.lambert_inputs(count=200 * 4096 + 3, dtype=dtype)
    assert x[0] == -30 and x[1] == 30
    t = torch.from_numpy(x.copy()).cuda()
    cuda_lib.lambert_w_exp_(t)
    y = t.cpu().numpy()
    y_ref = ref.prox("lambert_w_exp", x.reshape(1, -1)).ravel()
    tol = 1e-5 if dtype == np.float32 else 1e-12
    assert (np.abs(y - y_ref) <= tol * np.maximum(1, np.abs(y_ref))).all()
    # known answers of the reference's tests: W(exp(0)) = Omega; residuals
    z = torch.zeros(4, dtype=t.dtype, device="cuda")
    cuda_lib.lambert_w_exp_(z)
    assert abs(float(z[0]) - 0.5671432904097838) <= np.finfo(dtype).eps
    pos = x > 0
    w = y[pos].astype(np.float64)
    assert (np.abs(x[pos] - (w + np.log(w))) < 8 * np.finfo(dtype).eps * np.maximum(1, x[pos])).all()


def test_host_buffer_entry_point_matches_device_path(ref, cuda_lib):
    from libsdca_b200 import synth
    a = synth.topk_rows(rows=3000)
    x_host = cuda_lib.prox(a, "topk_simplex", k=5)
    x_dev = run_dev(cuda_lib, "topk_simplex", a, k=5)
    assert np.array_equal(x_host, x_dev)
    thr = cuda_lib.thresholds(a, "topk_simplex", k=5)
    assert len(thr) == 3000 and (thr["hi"] > 0).all()


def test_edge_shapes(ref, cuda_lib):
    rng = np.random.default_rng(3)
    # a single row, a single column, an odd number of rows, a row longer than
    # what fits in shared memory (read straight from global memory)
    for n, m in [(1, 7), (5, 1), (3, 70001)]:
        a = rng.standard_normal((n, m)).astype(np.float32)
        x = run_dev(cuda_lib, "knapsack", a)
        assert scaled_error(x, ref.prox("knapsack", a), a).max() <= 1e-5
        x = run_dev(cuda_lib, "topk_cone", a, k=1)
        assert scaled_error(x, ref.prox("topk_cone", a, k=1), a).max() <= 1e-5


@pytest.mark.parametrize("name", ["knapsack_eq", "knapsack_le", "knapsack_le_biased", "topk_simplex",
                                  "topk_simplex_biased"])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_accurate_math_matches_the_accurate_build(ref_accurate, cuda_lib, name, dtype):
    """opts.accurate_math = 1: the exact recomputation of t of the reference's
    SDCA_ACCURATE_MATH build (prox/knapsack_eq.h:87-106), against that build."""
    rng = np.random.default_rng(stable_seed("accurate-gpu", name, str(dtype)))
    for kind in ("normal", "pos", "neg", "mixed", "ties"):
        for m in (2, 5, 33, 100, 200, 1000, 1025):
            a = regime(rng, 37, m, dtype, kind)
            kw = random_opts(rng, name, m)
            x_ref = ref_accurate.prox(name, a, **kw)
            x = run_dev(cuda_lib, name, a, accurate_math=True, **kw)
            assert scaled_error(x, x_ref, a).max() <= tolerance(dtype, "double", m), (name, kind, m, kw)
