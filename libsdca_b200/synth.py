"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no dataset is involved: every configuration is
defined by its distribution and a seed).

All generators are numpy ``Generator(PCG64(seed))`` streams, so the CPU checkers
and the GPU path see identical bits.  ``rows`` lets tests take a prefix-sized
sample with the same construction.
"""
import numpy as np


def _rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def simplex_rows(rows=65536, m=100, seed=1):
    """Config 1: float64 N(0,1) rows for the simplex projection."""
    return _rng(seed).standard_normal((rows, m))


def topk_rows(rows=262144, m=1000, seed=2, tie_fraction=0.1, dtype=np.float32):
    """Config 2: float32 N(0,1) rows; ``tie_fraction`` of them get groups of 3-10
    exactly equal entries, one group always among the largest values so that
    ties straddle the top-k boundary."""
    rng = _rng(seed)
    a = rng.standard_normal((rows, m), dtype=np.float32).astype(dtype)
    tie_rows = np.nonzero(rng.random(rows) < tie_fraction)[0]
    for r in tie_rows:
        row = a[r]
        groups = int(rng.integers(1, 5))
        for g in range(groups):
            size = int(rng.integers(3, 11))
            size = min(size, m)
            idx = rng.choice(m, size=size, replace=False)
            if g == 0:
                # anchor the first group at one of the six largest entries
                top = np.argpartition(-row, min(5, m - 1))[:min(6, m)]
                idx[0] = top[int(rng.integers(0, len(top)))]
            row[idx] = row[idx[0]]
    return a


def entropy_rows(rows=1048576, m=200, seed=3, dtype=np.float32):
    """Config 3 projection inputs: N(0, 4), i.e. standard deviation 2."""
    rng = _rng(seed)
    a = rng.standard_normal((rows, m), dtype=np.float32)
    a *= np.float32(2.0)
    return a.astype(dtype)


def lambert_inputs(count=1048576 * 200, seed=4, dtype=np.float32):
    """Config 3 Lambert inputs: Uniform(-30, 30) with both endpoints present."""
    rng = _rng(seed)
    x = rng.random(count, dtype=np.float32)
    x = (x * np.float32(60.0) - np.float32(30.0)).astype(dtype)
    x[0] = -30.0
    if count > 1:
        x[1] = 30.0
    return x


def gap_problem(n=1048576, d=4096, m=1000, k=5, c=1.0, seed=5, dtype=np.float32, project=None):
    """Config 4: class-conditional Gaussian blobs and a random feasible dual point.

    Class means ~ N(0, I_d), labels uniform, x_i = mean[y_i] + 2 N(0, I_d).  The
    dual variables of example i are built the way an SDCA update leaves them
    (include/sdca/solver/objective/l2_hinge_topk.h:63-67 of the reference):
    v ~ N(0, 1)^(m-1) projected onto the top-k simplex of radius c, then
    a_ij = -v_j for j != y_i and a_iy = min(c, sum v).  ``project(v, k, rhs)``
    must return that projection (rows of v); W = X A' (d x m) is returned as its
    (m, d) row-major transpose, computed in float64 and rounded once.
    """
    rng = _rng(seed)
    means = rng.standard_normal((m, d), dtype=np.float32)
    labels = rng.integers(0, m, n).astype(np.int64)
    X = means[labels] + np.float32(2.0) * rng.standard_normal((n, d), dtype=np.float32)
    v = rng.standard_normal((n, m - 1), dtype=np.float32).astype(dtype)
    v = project(v, k, c)
    A = np.zeros((n, m), dtype=dtype)
    cols = np.arange(m - 1)[None, :] + (np.arange(m - 1)[None, :] >= labels[:, None])
    np.put_along_axis(A, cols, -v, axis=1)
    A[np.arange(n), labels] = np.minimum(c, v.astype(np.float64).sum(axis=1)).astype(dtype)
    X = X.astype(dtype)
    W = (A.astype(np.float64).T @ X.astype(np.float64)).astype(dtype)
    return X, A, W, labels


def kernel_problem(n=50000, dim=128, m=100, sigma=1.5, seed=6, dtype=np.float64):
    """Config 5: RBF Gram matrix of Gaussian blobs, gamma = 1 / dim."""
    rng = _rng(seed)
    means = rng.standard_normal((m, dim))
    labels = rng.integers(0, m, n).astype(np.int64)
    P = means[labels] + sigma * rng.standard_normal((n, dim))
    sq = (P * P).sum(axis=1)
    K = np.exp(-(sq[:, None] + sq[None, :] - 2.0 * (P @ P.T)).clip(min=0) / dim)
    return np.ascontiguousarray(K.astype(dtype)), labels
