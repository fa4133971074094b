// Threshold search of every proximal operator, written for one lane group per
// row.  Each routine returns the scalars (t, lo, hi) of
//     prox(a) = max(lo, min(map(a - t), hi))
// plus the sizes of the sets U (entries at hi) and M (entries strictly between
// the bounds), which is exactly what the reference's thresholds_<name>
// functions return (include/sdca/prox/proxdef.h:29-102 of the reference).
//
// Unlike the reference nothing is sorted, partitioned or copied: a row is only
// ever read, and every decision is taken from sums, counts and maxima over
// value ranges, which are butterfly reductions over the lanes of the group.
// A set is described by value cuts instead of iterator ranges:
//     {x > cutU}  is contained in U, which is contained in {x >= cutU}
//     {x > cutM}  is contained in U+M, which is contained in {x >= cutM}
// together with the counts nU and nM; entries equal to a cut fill the set up to
// its count.  Equal entries get equal outputs, so this is all that is needed.
//
// Comparisons and sums use the Result type, entries are stored as Data; that
// split is the reference's (e.g. include/sdca/prox/knapsack_eq.h:49-50).
#pragma once

#include <climits>

#include "math.cuh"
#include "warp.cuh"

namespace sdcab {

template <typename R>
struct Thr {
  R t, lo, hi;
  int nU, nM;
  R cutU, cutM;
  int status;   // 0: solved; kThrUnsettled: a bounded search ended without an admissible
                // answer and the all-zero default stands in (as in the reference)
};
enum { kThrSolved = 0, kThrUnsettled = 1, kThrNotFinite = 2 };

template <typename R>
SDCAB_HD Thr<R> make_thr(R t, R lo, R hi, int nU, int nM, R cutU, R cutM) {
  Thr<R> r;
  r.t = t; r.lo = lo; r.hi = hi; r.nU = nU; r.nM = nM; r.cutU = cutU; r.cutM = cutM;
  r.status = kThrSolved;
  return r;
}

// ---- row views -------------------------------------------------------------
// A view hands every lane its share of the row: for_each(f) calls
// f(value, index) with the value in Data precision.

template <typename Data>
struct StridedRow {
  typedef Data data_type;
  const Data* p;
  int m;
  SDCAB_HD StridedRow(const Data* p_, int m_) : p(p_), m(m_) {}
  SDCAB_D int size() const { return m; }
  template <typename F>
  SDCAB_D void for_each(F&& f) const {
    for (int i = lane_id(); i < m; i += kLanes) f(p[i], i);
  }
};

// The score vector of one example with the ground-truth entry left out and a
// constant added to the others, evaluated in Data precision; index i of the
// view is position i of the underlying vector (so m - 1 entries are visited).
template <typename Data>
struct ShiftedRow {
  typedef Data data_type;
  const Data* p;
  int m_all, skip;
  Data shift;
  SDCAB_HD ShiftedRow(const Data* p_, int m_all_, int skip_, Data shift_)
      : p(p_), m_all(m_all_), skip(skip_), shift(shift_) {}
  SDCAB_D int size() const { return m_all - 1; }
  template <typename F>
  SDCAB_D void for_each(F&& f) const {
    for (int i = lane_id(); i < m_all; i += kLanes)
      if (i != skip) f(static_cast<Data>(p[i] + shift), i);
  }
};

// ---- small reductions ------------------------------------------------------
template <typename R, typename Row>
SDCAB_D R row_sum(const Row& row) {
  R s = 0;
  row.for_each([&](typename Row::data_type x, int) { s += static_cast<R>(x); });
  return warp_sum(s);
}

// count and sum of the entries with x > cut
template <typename R, typename Row>
SDCAB_D void row_count_sum_gt(const Row& row, R cut, int& cnt, R& sum) {
  int c = 0; R s = 0;
  row.for_each([&](typename Row::data_type xd, int) {
    R x = static_cast<R>(xd);
    if (x > cut) { ++c; s += x; }
  });
  cnt = warp_sum(c); sum = warp_sum(s);
}

// Ordered extraction: the entries already taken are those that precede
// (v, idx) in the order "larger value first, smaller index first".
template <typename R>
struct Taken {
  R v;
  int idx;
  bool any;
  SDCAB_HD Taken() : v(0), idx(-1), any(false) {}
  SDCAB_HD bool has(R x, int i) const {
    return any && (x > v || (x == v && i <= idx));
  }
};

// Takes the largest entry not yet taken; false if none is left.
template <typename R, typename Row>
SDCAB_D bool take_next(const Row& row, Taken<R>& tk, R& val) {
  R best = -num<R>::inf();
  int bi = INT_MAX;
  row.for_each([&](typename Row::data_type xd, int i) {
    R x = static_cast<R>(xd);
    if (!tk.has(x, i) && (bi == INT_MAX || x > best)) { best = x; bi = i; }
  });
  // lanes without a candidate carry (-inf, INT_MAX) and lose every comparison
#if defined(__CUDA_ARCH__)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    R w = __shfl_xor_sync(kFullMask, best, o);
    int j = __shfl_xor_sync(kFullMask, bi, o);
    bool take = (j != INT_MAX) && (bi == INT_MAX || w > best || (w == best && j < bi));
    if (take) { best = w; bi = j; }
  }
#endif
  if (bi == INT_MAX) return false;
  tk.v = best; tk.idx = bi; tk.any = true;
  val = best;
  return true;
}

// ---- knapsack (continuous quadratic knapsack, variable fixing) -------------
// min 0.5<x,x> - <a,x>  s.t.  <1,x> = rhs, lo <= x <= hi.
// Same iteration as include/sdca/prox/knapsack_eq.h:25-109 (Kiwiel's variable
// fixing): the free entries always form a value interval (lb, ub], so fixing a
// tail moves one end of the interval instead of partitioning the data.
// The exact recomputation of t that the reference makes when it is compiled with
// SDCA_ACCURATE_MATH (include/sdca/prox/knapsack_eq.h:87-106): from the final sets,
// t = (sum of the middle entries - rhs + hi |U| + lo |L|) / |M|, kept between
// max(L) - lo and min(U) - hi; their midpoint when M is empty.
template <typename R, typename Row>
SDCAB_D Thr<R> knapsack_recompute_t(const Row& row, Thr<R> thr, R rhs) {
  const int m = row.size();
  R sum_M = 0, max_L = -num<R>::inf(), min_U = num<R>::inf();
  int nU = 0, nM = 0;
  row.for_each([&](typename Row::data_type xd, int) {
    const R x = static_cast<R>(xd);
    if (x > thr.cutU) { ++nU; min_U = min_(min_U, x); }
    else if (x > thr.cutM) { ++nM; sum_M += x; }
    else max_L = max_(max_L, x);
  });
  sum_M = warp_sum(sum_M); max_L = warp_max(max_L); min_U = -warp_max(-min_U);
  nU = warp_sum(nU); nM = warp_sum(nM);
  const int nL = m - nU - nM;
  const R t_lo = (nL > 0) ? max_L - thr.lo : -num<R>::max();
  const R t_hi = (nU > 0) ? min_U - thr.hi : num<R>::max();
  R t;
  if (nM > 0) {
    t = (sum_M - rhs + thr.hi * static_cast<R>(nU) + thr.lo * static_cast<R>(nL)) / static_cast<R>(nM);
    t = max_(t_lo, min_(t, t_hi));
  } else {
    t = R(0.5) * (t_lo + t_hi);
  }
  thr.t = t;
  return thr;
}

template <typename R, typename Row>
SDCAB_D Thr<R> thr_knapsack_eq(const Row& row, R lo, R hi, R rhs, bool accurate = false) {
  const int m = row.size();
  const R eps = num<R>::eps() * max_(R(1), abs_(rhs));
  const R total = row_sum<R>(row);
  int mfree = m, nU_fixed = 0;
  R t = (total - rhs) / static_cast<R>(m);
  R lb = -num<R>::inf(), ub = num<R>::inf();
  for (int it = 0;; ++it) {
    const R tlo = lo + t, thi = hi + t;
    R sum_lo = 0, sum_hi = 0;
    int n_lo = 0, n_hi = 0;
    row.for_each([&](typename Row::data_type xd, int) {
      R x = static_cast<R>(xd);
      if (x > lb && x <= ub) {
        if (x > tlo) {
          if (x > thi) { sum_hi += x; ++n_hi; }
        } else {
          sum_lo += x; ++n_lo;
        }
      }
    });
    sum_lo = warp_sum(sum_lo); sum_hi = warp_sum(sum_hi);
    n_lo = warp_sum(n_lo); n_hi = warp_sum(n_hi);
    const R s_hi = static_cast<R>(n_hi) * hi, s_lo = static_cast<R>(n_lo) * lo;
    const R infeas = sum_hi + sum_lo - (s_hi + s_lo) - static_cast<R>(n_hi + n_lo) * t;
    R tt;
    if (n_hi > 0 && infeas > eps && it <= m) {
      ub = min_(ub, thi);
      tt = static_cast<R>(mfree) * t - sum_hi + s_hi;
      mfree -= n_hi; nU_fixed += n_hi;
    } else if (n_lo > 0 && infeas < -eps && it <= m) {
      lb = max_(lb, tlo);
      tt = static_cast<R>(mfree) * t - sum_lo + s_lo;
      mfree -= n_lo;
    } else {
      const Thr<R> thr = make_thr(t, lo, hi, nU_fixed + n_hi, mfree - n_hi - n_lo,
                                  min_(ub, thi), max_(lb, tlo));
      return accurate ? knapsack_recompute_t<R>(row, thr, rhs) : thr;
    }
    if (mfree > 0) {
      t = tt / static_cast<R>(mfree);
    } else {
      // everything is fixed: the entries above ub sit at hi, the others at lo
      const Thr<R> thr = make_thr(t, lo, hi, nU_fixed, 0, ub, ub);
      return accurate ? knapsack_recompute_t<R>(row, thr, rhs) : thr;
    }
  }
}

// <1,x> <= rhs                   (include/sdca/prox/knapsack_le.h:17-44)
template <typename R, typename Row>
SDCAB_D Thr<R> thr_knapsack_le(const Row& row, R lo, R hi, R rhs, bool accurate = false) {
  const R eps = num<R>::eps() * max_(R(1), abs_(rhs));
  int n_hi = 0, n_mid = 0;
  R sum_mid = 0;
  row.for_each([&](typename Row::data_type xd, int) {
    R x = static_cast<R>(xd);
    if (x >= hi) ++n_hi;
    else if (x > lo) { ++n_mid; sum_mid += x; }
  });
  n_hi = warp_sum(n_hi); n_mid = warp_sum(n_mid); sum_mid = warp_sum(sum_mid);
  const int n_lo = row.size() - n_hi - n_mid;
  const R s = sum_mid + hi * static_cast<R>(n_hi) + lo * static_cast<R>(n_lo);
  if (s > rhs + eps) return thr_knapsack_eq<R>(row, lo, hi, rhs, accurate);
  return make_thr(R(0), lo, hi, n_hi, n_mid, hi, lo);
}

// Solves rho * sum_i clip(a_i - t, lo, hi) = t.  The left side is piecewise
// linear and decreasing in t, so the step "solve on the current piece" is a
// Newton step; a bracket guards against cycling on the non-convex parts.
template <typename R, typename Row>
SDCAB_D Thr<R> thr_knapsack_le_biased_root(const Row& row, R lo, R hi, R rhs, R rho, R t0) {
  const int m = row.size();
  const R eps = num<R>::eps() * max_(R(1), abs_(rhs));
  const R rho_inv = R(1) / rho;
  R t = t0, tl = -num<R>::inf(), tr = num<R>::inf();
  int pU = -1, pM = -1;
  int nU = 0, nM = 0;
  bool newton = false;  // t is the root of the previous piece's line
  for (int it = 0; it < 2 * m + 128; ++it) {
    const R tlo = lo + t, thi = hi + t;
    int cU = 0, cM = 0; R sM = 0;
    row.for_each([&](typename Row::data_type xd, int) {
      R x = static_cast<R>(xd);
      if (x > thi) ++cU;
      else if (x > tlo) { ++cM; sM += x; }
    });
    nU = warp_sum(cU); nM = warp_sum(cM); sM = warp_sum(sM);
    const R base = lo * static_cast<R>(m - nU - nM) + hi * static_cast<R>(nU) + sM;
    const R f = rho * (base - static_cast<R>(nM) * t) - t;
    if (f > 0) tl = max_(tl, t); else tr = min_(tr, t);
    R tn = base / (rho_inv + static_cast<R>(nM));
    // t solves the line of the piece it lies on: done
    if ((newton && nU == pU && nM == pM) || tn == t) { t = tn; break; }
    pU = nU; pM = nM;
    newton = (tn > tl && tn < tr) || !(finite_(tl) && finite_(tr));
    if (!newton) {
      tn = R(0.5) * (tl + tr);
      if (!(tn > tl && tn < tr)) break;  // bracket exhausted
    }
    t = tn;
  }
  if (!(t <= rho * rhs + eps)) {
    Thr<R> none = make_thr(R(0), R(0), R(0), 0, 0, R(0), R(0));
    none.status = kThrUnsettled;
    return none;
  }
  return make_thr(t, lo, hi, nU, nM, hi + t, lo + t);
}

// min 0.5(<x,x> + rho<1,x>^2) - <a,x>,  <1,x> <= rhs,  lo <= x <= hi
// (include/sdca/prox/knapsack_le_biased.h:106-129; the sorted double loop of
//  :10-86 is replaced by the one-dimensional root search above)
template <typename R, typename Row>
SDCAB_D Thr<R> thr_knapsack_le_biased(const Row& row, R lo, R hi, R rhs, R rho, bool accurate = false) {
  if (rho == 0) return thr_knapsack_le<R>(row, lo, hi, rhs, accurate);
  const R eps = num<R>::eps() * max_(R(1), abs_(rhs));
  Thr<R> eq = thr_knapsack_eq<R>(row, lo, hi, rhs, accurate);
  if (eq.t >= rho * rhs - eps) return eq;
  return thr_knapsack_le_biased_root<R>(row, lo, hi, rhs, rho, eq.t);
}

// ---- top-k cone / simplex ---------------------------------------------------
enum Projection { kProjZero = 0, kProjConstant = 1, kProjGeneral = 2 };

// Zero / constant / general classification
// (include/sdca/prox/topk_cone.h:18-55).
template <typename R, typename Row>
SDCAB_D Projection topk_special_cases(const Row& row, int k, R div, Thr<R>& thr) {
  const R eps = 16 * num<R>::eps();
  Taken<R> tk;
  R sum_k = 0, v_k = 0;
  for (int j = 0; j < k; ++j) {
    R v;
    take_next<R>(row, tk, v);
    sum_k += v; v_k = v;
  }
  if (sum_k <= eps) {
    thr = make_thr(R(0), R(0), R(0), 0, 0, num<R>::inf(), num<R>::inf());
    return kProjZero;
  }
  const R hi = sum_k / div;
  const R t = v_k - hi;
  bool constant = (k == row.size());
  if (!constant) {
    R nxt;
    Taken<R> peek = tk;
    take_next<R>(row, peek, nxt);
    constant = (t >= nxt - eps);
  }
  if (constant) {
    thr = make_thr(t, R(0), hi, k, 0, v_k, v_k);
    return kProjConstant;
  }
  return kProjGeneral;
}

// min 0.5(<x,x> + rho<1,x>^2) - <a,x>,  0 <= x_i <= <1,x>/k   (rho = 0: plain)
//
// The reference sorts the row and scans |U| = 0..k (outer) and |M| = 0..
// (inner) for the first pair whose closed-form (t, hi) passes four inequalities
// (include/sdca/prox/topk_cone.h:58-133, topk_cone_biased.h:8-113).  For a fixed
// U the pair (M, t) is the root of a convex decreasing piecewise-linear
// function, reached here from the left by Newton steps on the set
// M = {non-U entries > t}; only the checks that tie U to M remain.
template <typename R, typename Row>
SDCAB_D Thr<R> thr_topk_cone_search(const Row& row, int k, R rho) {
  const int m = row.size();
  const R K = static_cast<R>(k);
  const R rho_k2 = rho * K * K;
  const R eps = 16 * num<R>::eps();
  const R total = row_sum<R>(row);
  Taken<R> tk;
  R sum_U = 0, min_U = num<R>::inf();
  for (int u = 0; u <= k; ++u) {
    const R kmu = K - static_cast<R>(u), up = static_cast<R>(u) + rho_k2;
    Taken<R> nx = tk;
    R s_u = 0;
    const bool has_next = take_next<R>(row, nx, s_u);
    int j = 0; R sum_M = 0;
    bool valid = true;
    if (u == k) {
      // D = up * |M|: the only admissible M is the single next entry
      if (has_next && up > 0) { j = 1; sum_M = s_u; } else valid = false;
    } else {
      j = m - u; sum_M = total - sum_U;
      for (int it = 0; it <= m; ++it) {
        const R D = kmu * kmu + up * static_cast<R>(j);
        const R t = (up * sum_M - kmu * sum_U) / D;
        int c = 0; R s = 0;
        row.for_each([&](typename Row::data_type xd, int i) {
          R x = static_cast<R>(xd);
          if (x > t && !tk.has(x, i)) { ++c; s += x; }
        });
        c = warp_sum(c); s = warp_sum(s);
        if (c == j) break;
        j = c; sum_M = s;
      }
    }
    if (valid) {
      const R D = kmu * kmu + up * static_cast<R>(j);
      const R t = (up * sum_M - kmu * sum_U) / D;
      const R hi = (static_cast<R>(j) * sum_U + kmu * sum_M) / D;
      const R tt = hi + t;
      const R max_M = (j > 0) ? s_u : -num<R>::inf();
      if (max_M - eps <= tt && tt <= min_U + eps) {
        bool ok = true;
        if (u == k) ok = (t <= s_u + eps);
        else if (j == 0 && has_next) ok = (s_u - eps <= t);
        if (ok) {
          return make_thr(t, R(0), hi, u, j, min_U, (j > 0) ? t : min_U);
        }
      }
    }
    if (!has_next) break;
    tk = nx; min_U = s_u; sum_U += s_u;
  }
  Thr<R> none = make_thr(R(0), R(0), R(0), 0, 0, num<R>::inf(), num<R>::inf());
  none.status = kThrUnsettled;
  return none;
}

// (include/sdca/prox/topk_cone.h:144-157, topk_cone_biased.h:124-139)
template <typename R, typename Row>
SDCAB_D Thr<R> thr_topk_cone(const Row& row, int k, R rho) {
  const R K = static_cast<R>(k);
  Thr<R> thr;
  if (topk_special_cases<R>(row, k, K + rho * K * K, thr) == kProjGeneral)
    return thr_topk_cone_search<R>(row, k, rho);
  return thr;
}

// min 0.5(<x,x> + rho<1,x>^2) - <a,x>,  <1,x> <= rhs,  0 <= x_i <= <1,x>/k
// (include/sdca/prox/topk_simplex.h:9-68, topk_simplex_biased.h:9-71)
template <typename R, typename Row>
SDCAB_D Thr<R> thr_topk_simplex(const Row& row, int k, R rhs, R rho, bool accurate = false) {
  const R K = static_cast<R>(k), lo = 0;
  const R eps = num<R>::eps() * max_(R(1), abs_(rhs));
  const R rho_k2 = rho * K * K;
  Thr<R> thr;
  const Projection proj = topk_special_cases<R>(row, k, K + rho_k2, thr);
  if (proj == kProjZero) return thr;
  if (proj == kProjConstant) {
    if (K * thr.hi > rhs + eps) return thr_knapsack_eq<R>(row, lo, rhs / K, rhs, accurate);
    return thr;
  }
  Thr<R> eq = thr_knapsack_eq<R>(row, lo, rhs / K, rhs, accurate);
  bool lt;
  if (eq.nU == 0) {
    lt = eq.t < rho * rhs - eps;
  } else {
    int cnt; R sum_U;
    row_count_sum_gt<R>(row, eq.cutU, cnt, sum_U);
    const R num_U = static_cast<R>(cnt);
    lt = K * (sum_U + (K - num_U) * eq.t) < rhs * (num_U + rho_k2) - eps;
  }
  if (lt) return thr_topk_cone_search<R>(row, k, rho);
  return eq;
}

// ---- entropic projections ---------------------------------------------------
// log(sum exp) over the entries selected by `in`, shifted by their maximum and
// with one instance of the maximum left out of the sum, as in
// include/sdca/math/log_exp.h:88-103.  Returns the maximum in mx, the sum of
// the other terms in s; count is the number of selected entries.
template <typename R, typename Row, typename Pred>
SDCAB_D void row_max_sumexp(const Row& row, Pred in, R& mx, R& s, int& count) {
  R best = -num<R>::inf();
  int bi = INT_MAX, c = 0;
  row.for_each([&](typename Row::data_type xd, int i) {
    R x = static_cast<R>(xd);
    if (in(x, i)) {
      ++c;
      if (bi == INT_MAX || x > best) { best = x; bi = i; }
    }
  });
#if defined(__CUDA_ARCH__)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    R w = __shfl_xor_sync(kFullMask, best, o);
    int j = __shfl_xor_sync(kFullMask, bi, o);
    bool take = (j != INT_MAX) && (bi == INT_MAX || w > best || (w == best && j < bi));
    if (take) { best = w; bi = j; }
  }
#endif
  count = warp_sum(c);
  R acc = 0;
  row.for_each([&](typename Row::data_type xd, int i) {
    R x = static_cast<R>(xd);
    if (i != bi && in(x, i)) acc += exp_(x - best);
  });
  mx = best;
  s = warp_sum(acc);
}

// min <x,log x> - <a,x>,  <1,x> = rhs,  0 <= x <= hi; x = min(exp(a - t), hi)
// (include/sdca/prox/entropy.h:19-53)
template <typename R, typename Row>
SDCAB_D Thr<R> thr_entropy(const Row& row, R hi, R rhs) {
  const int m = row.size();
  const R eps = 16 * num<R>::eps() * max_(R(1), rhs);
  const R u = log_(hi) + eps;
  R r = rhs;
  R cut = num<R>::inf();  // free entries: x <= cut
  int nU = 0;
  R mx, s; int cnt;
  row_max_sumexp<R>(row, [&](R, int) { return true; }, mx, s, cnt);
  R t = (mx + log1p_(s)) - log_(rhs);
  for (int it = 0; it <= m; ++it) {
    const R tt = t + u;
    int c = 0;
    row.for_each([&](typename Row::data_type xd, int) {
      R x = static_cast<R>(xd);
      if (x <= cut && x > tt) ++c;
    });
    c = warp_sum(c);
    if (c == 0) break;
    r -= hi * static_cast<R>(c);
    nU += c;
    cut = min_(cut, tt);
    if (nU == m) break;
    row_max_sumexp<R>(row, [&](R x, int) { return x <= cut; }, mx, s, cnt);
    if (r <= eps) {
      t = mx - num<R>::exp_min_arg() + 1;
      break;
    }
    t = (mx + log1p_(s)) - log_(r);
  }
  return make_thr(t, R(0), hi, nU, m - nU, cut, -num<R>::inf());
}

// min <x,log x> + (1-s)log(1-s) - <a,x>,  <1,x> = s <= 1,  0 <= x_i <= s/k
// (include/sdca/prox/topk_entropy.h:20-76)
template <typename R, typename Row>
SDCAB_D Thr<R> thr_topk_entropy(const Row& row, int k) {
  const int m = row.size();
  const R eps = 16 * num<R>::eps();
  const R K = static_cast<R>(k);
  R mx, z; int cnt;
  row_max_sumexp<R>(row, [&](R, int) { return true; }, mx, z, cnt);
  R log_z = mx + log1p_(z);
  R e = exp_(-mx);
  const R log_z_1 = finite_(e) ? mx + log1p_(z + e) : R(0);
  if (k <= 1 || mx - eps <= log_z - log_(K)) {
    return make_thr(log_z_1, R(0), R(1), 0, m, num<R>::inf(), -num<R>::inf());
  }
  // U grows by the largest remaining entry until the bound is consistent
  Taken<R> tk;
  R min_U = 0, sum_U = 0, k_u = K;
  int num_U = 0;
  R cur_max = mx;  // maximum of the entries not in U
  for (num_U = 1; num_U < k; ++num_U) {
    R v;
    take_next<R>(row, tk, v);  // v == cur_max
    min_U = v; sum_U += v; k_u -= 1;
    row_max_sumexp<R>(row, [&](R x, int i) { return !tk.has(x, i); }, cur_max, z, cnt);
    log_z = cur_max + log1p_(z);
    const R tt = log_z - log_(k_u);
    if (cur_max - eps <= tt && tt <= min_U + eps) break;
  }
  // after the loop |U| = K - k_u (the loop may end without a break)
  const int nU = static_cast<int>(K - k_u);
  const R tmp = ((K - k_u) * log_z + k_u * log_(k_u) - sum_U) / K;
  R t, hi;
  if (tmp > cur_max) {
    const R a = (1 + z) * exp_(cur_max - tmp);
    t = tmp + log1p_(a * K) - log_(k_u);
    hi = a / (1 + a * K);
  } else {
    const R a = exp_(tmp - cur_max) / K;
    t = cur_max + log1p_(z + a) - log_(k_u / K);
    hi = (1 + z) / ((1 + z + a) * K);
  }
  return make_thr(t, R(0), hi, nU, m - nU, min_U, -num<R>::inf());
}

// ---- Lambert-W based projections --------------------------------------------
// f0 = sum W(exp(a_i - t)) and its first three derivative sums over the
// entries selected by `in` (include/sdca/math/lambert.h:224-332).
template <typename R, typename Row, typename Pred>
SDCAB_D void row_sum_w_exp(const Row& row, Pred in, R t, int order, R& f0, R& f1,
                           R& f2, R& f3) {
  R a0 = 0, a1 = 0, a2 = 0, a3 = 0;
  row.for_each([&](typename Row::data_type xd, int i) {
    R x = static_cast<R>(xd);
    if (!in(x, i)) return;
    const R v = lambert_w_exp(x - t);
    const R d = 1 + v;
    a0 += v;
    a1 += v / d;
    if (order >= 3) {
      const R d3 = d * d * d;
      a2 += v / d3;
      a3 += v * (1 - 2 * v) / (d3 * d * d);
    }
  });
  f0 = warp_sum(a0); f1 = warp_sum(a1);
  if (order >= 3) { f2 = warp_sum(a2); f3 = warp_sum(a3); } else { f2 = 0; f3 = 0; }
}

// Root of sum_i W(exp(a_i - t)) = rhs over the selected entries
// (include/sdca/prox/entropy_norm.h:80-134): the linear heuristic for the
// start, then fourth-order Householder steps.
template <typename R, typename Row, typename Pred>
SDCAB_D R solve_sum_w_exp(const Row& row, Pred in, R rhs) {
  // start: t = (sum_{a > t} a - rhs) / |{a > t}|, iterated while the set shrinks
  R sum = 0; int cnt = 0;
  R amax = -num<R>::inf();
  row.for_each([&](typename Row::data_type xd, int i) {
    R x = static_cast<R>(xd);
    if (in(x, i)) { sum += x; ++cnt; amax = max_(amax, x); }
  });
  sum = warp_sum(sum); cnt = warp_sum(cnt); amax = warp_max(amax);
  R t = (sum - rhs) / static_cast<R>(cnt);
  int prev = cnt;
  for (int it = 0; it <= row.size(); ++it) {
    R s = 0; int c = 0;
    row.for_each([&](typename Row::data_type xd, int i) {
      R x = static_cast<R>(xd);
      if (in(x, i) && x > t) { s += x; ++c; }
    });
    s = warp_sum(s); c = warp_sum(c);
    if (c == prev || c == 0) break;
    prev = c;
    t = (s - rhs) / static_cast<R>(c);
  }
  // Householder iterations with the underflow guard t <= max - min_arg
  const R ub = amax - num<R>::exp_min_arg();
  const R eps = 16 * num<R>::eps();
  for (int iter = 0; iter < 32; ++iter) {
    const R t1 = t;
    const R tc = min_(t, ub);
    R f0, f1, f2, f3;
    row_sum_w_exp<R>(row, in, tc, 3, f0, f1, f2, f3);
    f0 -= rhs;
    const R f02 = f0 * f2, f11 = f1 * f1;
    t = tc - 3 * f0 * (2 * f11 - f02) / (6 * f1 * (f02 - f11) - f0 * (f0 * f3));
    if (abs_(t1 - t) <= eps) break;
  }
  return t;
}

template <typename R>
struct ThrPair { Thr<R> a, b; };

// A view of a single entry (the label's block of a multiclass example).
template <typename Data>
struct OneEntryRow {
  typedef Data data_type;
  Data x;
  int index;
  SDCAB_D int size() const { return 1; }
  template <typename F>
  SDCAB_D void for_each(F&& f) const {
    if (lane_id() == 0) f(x, index);
  }
};

// min over two blocks x, y >= 0 with <1,x> + <1,y> = 1 of the entropic objectives
// of include/sdca/prox/two_entropy.h:94-231: x = W(exp(a - t)) / alpha,
// y = W(exp(b - t - c)) / alpha with c = alpha / |a|, t the root of
//   F(t) = sum_i W(exp(a_i - t)) + sum_j W(exp(b_j - t - c)) - alpha.
// Same course as the reference: two starting guesses (the function taken as an
// exponential, and as linear), one Householder step from each to bracket the root,
// a few bisections if they bracket it, then Householder steps kept inside the
// bracket.  Returns the thresholds of the two blocks (t and t + c; lo 0, hi 1).
template <typename R, typename RowA, typename RowB>
SDCAB_D ThrPair<R> thr_two_entropy(const RowA& ra, const RowB& rb, R alpha) {
  const R num_a = static_cast<R>(ra.size()), num_b = static_cast<R>(rb.size());
  R max_a = -num<R>::inf(), max_b = -num<R>::inf(), sum_a = 0, sum_b = 0;
  ra.for_each([&](typename RowA::data_type xd, int) { const R x = static_cast<R>(xd); max_a = max_(max_a, x); sum_a += x; });
  rb.for_each([&](typename RowB::data_type xd, int) { const R x = static_cast<R>(xd); max_b = max_(max_b, x); sum_b += x; });
  max_a = warp_max(max_a); max_b = warp_max(max_b);
  sum_a = warp_sum(sum_a); sum_b = warp_sum(sum_b);
  const R c = alpha / num_a;
  const R mx = max_(max_a, max_b - c);
  const R eps = num<R>::eps();
  auto all = [](R, int) { return true; };
  // F(t) (without the derivatives)
  auto value = [&](R t) {
    R f0, f1, f2, f3, g0, g1, g2, g3;
    row_sum_w_exp<R>(ra, all, t, 1, f0, f1, f2, f3);
    row_sum_w_exp<R>(rb, all, t + c, 1, g0, g1, g2, g3);
    return f0 + g0 - alpha;
  };
  // one Householder step of order four at t; returns F(t) (two_entropy.h:12-37)
  auto step = [&](R& t) {
    R f0, f1, f2, f3, g0, g1, g2, g3;
    row_sum_w_exp<R>(ra, all, t, 3, f0, f1, f2, f3);
    row_sum_w_exp<R>(rb, all, t + c, 3, g0, g1, g2, g3);
    f0 += g0; f1 += g1; f2 += g2; f3 += g3;
    f0 -= alpha;
    const R f02 = f0 * f2, f11 = f1 * f1;
    const R D = 6 * f1 * (f02 - f11) - f0 * (f0 * f3);
    if (abs_(D) > 64 * num<R>::tiny()) t -= 3 * f0 * (2 * f11 - f02) / D;
    return f0;
  };
  R lb = -num<R>::max(), ub = mx - 64 * num<R>::exp_min_arg();
  R lf = num<R>::max(), uf = -num<R>::max();
  R t01 = mx - log_(alpha), t1 = t01;
  R f1v = step(t1);
  R t02 = (sum_a + sum_b - num_b * c - alpha) / (num_a + num_b), t2 = t02;
  R f2v = step(t2);
  if (f1v > f2v) {
    R tmp = t01; t01 = t02; t02 = tmp;
    tmp = t1; t1 = t2; t2 = tmp;
    tmp = f1v; f1v = f2v; f2v = tmp;
  }
  R t;
  if (f1v > 0) {
    lb = t01; lf = f1v; t = t1;
  } else if (f2v < 0) {
    ub = t02; uf = f2v; t = t2;
  } else {
    lb = t02; ub = t01; lf = f2v; uf = f1v;
    t = max_(lb, min_(abs_(f1v) < abs_(f2v) ? t1 : t2, ub));
    // a few bisections to improve the guess (two_entropy.h:63-91,198-203)
    const R width = log_(ub - lb) * R(1.4426950408889634);
    int num_iter = 0;
    if (width > 0) num_iter = width < R(32) ? static_cast<int>(width) : 32;
    for (int iter = 0; iter < num_iter; ++iter) {
      t = (lb + ub) / 2;
      const R fm = value(t);
      if (eps < fm && fm < lf) { lf = fm; lb = t; }
      else if (uf < fm && fm < -eps) { uf = fm; ub = t; }
      else break;
    }
    t = (lb + ub) / 2;
  }
  for (int iter = 0; iter < 32; ++iter) {
    const R tb = t;
    const R fv = step(t);
    if (0 <= fv && fv < lf) { lb = tb; lf = fv; }
    else if (uf < fv && fv <= 0) { ub = tb; uf = fv; }
    t = max_(lb, min_(t, ub));
    if (abs_(tb - t) <= eps) break;
  }
  ThrPair<R> out;
  out.a = make_thr(t, R(0), R(1), 0, ra.size(), num<R>::inf(), -num<R>::inf());
  out.b = make_thr(t + c, R(0), R(1), 0, rb.size(), num<R>::inf(), -num<R>::inf());
  return out;
}

// min 0.5<x,x> + <x,log x> - <a,x>,  <1,x> = rhs,  0 <= x <= hi;
// x = min(W(exp(a - t)), hi)        (include/sdca/prox/entropy_norm.h:146-181)
template <typename R, typename Row>
SDCAB_D Thr<R> thr_entropy_norm(const Row& row, R hi, R rhs) {
  const int m = row.size();
  const R eps = 16 * num<R>::eps() * max_(R(1), rhs);
  const R u = hi + log_(hi) + eps;
  R r = rhs;
  R cut = num<R>::inf();
  int nU = 0;
  R t = solve_sum_w_exp<R>(row, [&](R, int) { return true; }, rhs);
  for (int it = 0; it <= m; ++it) {
    const R tt = t + u;
    int c = 0;
    row.for_each([&](typename Row::data_type xd, int) {
      R x = static_cast<R>(xd);
      if (x <= cut && x > tt) ++c;
    });
    c = warp_sum(c);
    if (c == 0) break;
    r -= hi * static_cast<R>(c);
    nU += c;
    cut = min_(cut, tt);
    if (nU == m) break;
    if (r <= eps) {
      R mx = -num<R>::inf();
      row.for_each([&](typename Row::data_type xd, int) {
        R x = static_cast<R>(xd);
        if (x <= cut) mx = max_(mx, x);
      });
      mx = warp_max(mx);
      t = mx - num<R>::exp_min_arg() + 1;
      break;
    }
    t = solve_sum_w_exp<R>(row, [&](R x, int) { return x <= cut; }, r);
  }
  return make_thr(t, R(0), hi, nU, m - nU, cut, -num<R>::inf());
}

// min 0.5 alpha(<x,x> + s^2) + <x,log x> + (1-s)log(1-s) - <a,x>,
//     <1,x> = s <= 1,  0 <= x_i <= s/k;   x = min(W(exp(a - t))/alpha, hi)
// (include/sdca/prox/topk_entropy_biased.h:15-270)
template <typename R, typename Row>
SDCAB_D Thr<R> thr_topk_entropy_biased(const Row& row, int k, R alpha) {
  const int m = row.size();
  R mx = -num<R>::inf();
  row.for_each([&](typename Row::data_type xd, int) { mx = max_(mx, static_cast<R>(xd)); });
  mx = warp_max(mx);
  const R eps = 16 * num<R>::eps() * max_(R(1), mx);
  const R K = static_cast<R>(k), lo = 0;
  const R tiny64 = 64 * num<R>::tiny();
  R s = 0, t = mx;
  // U empty: W(exp(alpha - t)) + sum_i W(exp(a_i - t)) = alpha   (:15-64)
  {
    const R e1 = num<R>::eps();
    for (int iter = 0; iter < 32; ++iter) {
      const R t1 = t;
      R f0, f1, f2, f3;
      row_sum_w_exp<R>(row, [&](R, int) { return true; }, t, 3, f0, f1, f2, f3);
      s = f0 / alpha;
      {
        const R v = lambert_w_exp(alpha - t);
        const R d = 1 + v, d3 = d * d * d;
        f0 += v; f1 += v / d; f2 += v / d3; f3 += v * (1 - 2 * v) / (d3 * d * d);
      }
      f0 -= alpha;
      const R f02 = f0 * f2, f11 = f1 * f1;
      const R D = 6 * f1 * (f02 - f11) - f0 * (f0 * f3);
      if (abs_(D) > tiny64) t -= 3 * f0 * (2 * f11 - f02) / D;
      if (abs_(t1 - t) <= e1) break;
    }
  }
  if (k == 1) return make_thr(t, lo, s, 0, m, num<R>::inf(), -num<R>::inf());

  const R alpha_k = alpha / K;
  R tt = t + max_(lambert_w_exp_inverse(alpha_k * s), num<R>::exp_min_arg());
  if (mx - eps <= tt) return make_thr(t, lo, s / K, 0, m, num<R>::inf(), -num<R>::inf());

  // U not empty: grow it by the largest remaining entry; for each size solve
  // the two-dimensional KKT system in (s, t) by Newton steps   (:72-175)
  const R log_k = log_(K), log_alpha = log_(alpha);
  Taken<R> tk;
  R v;
  take_next<R>(row, tk, v);
  R min_U = v, sum_U = v;
  int num_U = 1;
  const R eps16 = 16 * num<R>::eps();
  for (; num_U < m;) {
    Taken<R> nx = tk;
    R cur;
    take_next<R>(row, nx, cur);  // largest entry outside U
    const R U = static_cast<R>(num_U);
    s = R(0.999); t = cur;
    const R C1 = U * K;
    const R C2 = (K + U) * alpha;
    const R C3 = (K - U) * (U - 1) * alpha;
    const R C4 = K * (U - 1);
    const R C5 = (1 - U / K) * alpha;
    const R C0 = C4 * log_alpha - C1 * log_k - sum_U;
    for (int iter = 0; iter < 32; ++iter) {
      const R s1 = s, t1 = t;
      s = min_(max_(R(0), s), R(1));
      R S0, S1, d2, d3;
      row_sum_w_exp<R>(row, [&](R x, int i) { return !tk.has(x, i); }, t, 1, S0, S1, d2, d3);
      const R E = S0 + t * S1;
      R z, Az, Bz;
      if (s < R(0.5)) {
        z = s;
        Az = K * (z * (U + log1p_(-z) + z / (1 - z)) - U * x_log_x(z)) - C0 * z;
        Bz = z * (C2 + K / (1 - z)) + C1;
      } else {
        z = 1 - s;
        Az = K * (z * (U - U * log1p_(-z) - 1) + x_log_x(z) + 1) - C0 * z;
        Bz = z * (C2 + C1 / (1 - z)) + K;
      }
      const R Dz = C3 * z - Bz * S1;
      if (abs_(Dz) > tiny64) {
        s = (C4 * E * z - Az * S1) / Dz;
        t = (C5 * Az - E * Bz) / Dz;
      }
      if (abs_(s1 - s) + abs_(t1 - t) <= eps16) break;
    }
    s = min_(max_(R(0), s), R(1));
    tt = t + max_(lambert_w_exp_inverse(alpha_k * s), num<R>::exp_min_arg());
    if (cur - eps <= tt && tt <= min_U + eps) break;
    if (++num_U > k) break;
    tk = nx; min_U = cur; sum_U += cur;
  }
  // the reference reports every entry as "middle" for this operator
  return make_thr(t, lo, s / K, 0, m, num<R>::inf(), -num<R>::inf());
}

// ---- bipartite simplex ------------------------------------------------------
// min ||x-a||^2 + ||y-b||^2,  <1,x> = <1,y> <= rhs,  x, y >= 0
// (include/sdca/prox/two_simplex.h:18-119).  Returns the pair (t for a, s for b).


template <typename R, typename Row>
SDCAB_D void simplex_phase1(const Row& row, R rhs, R& t, int& n_active, R& cut) {
  // t = (sum_{x in X} x - rhs)/|X|, X <- {x in X : x > t} until X is stable
  cut = -num<R>::inf();
  int prev = row.size();
  R sum = row_sum<R>(row);
  for (int it = 0;; ++it) {
    t = (sum - rhs) / static_cast<R>(prev);
    int c; R s;
    row_count_sum_gt<R>(row, max_(cut, t), c, s);
    if (c == prev || it > row.size()) break;
    cut = max_(cut, t);
    prev = c; sum = s;
    if (c == 0) break;
  }
  n_active = prev;
}

template <typename R, typename RowA, typename RowB>
SDCAB_D ThrPair<R> thr_two_simplex(const RowA& ra, const RowB& rb, R rhs) {
  const R lo = 0, hi = rhs;
  const R eps = num<R>::eps() * max_(R(1), rhs);
  R t, s, cut_x, cut_y;
  int nx, ny;
  simplex_phase1<R>(ra, rhs, t, nx, cut_x);
  simplex_phase1<R>(rb, rhs, s, ny, cut_y);
  ThrPair<R> out;
  if (t + s >= -eps) {
    out.a = make_thr(t, lo, hi, 0, nx, num<R>::inf(), cut_x);
    out.b = make_thr(s, lo, hi, 0, ny, num<R>::inf(), cut_y);
    return out;
  }
  // phase 2: <1,x> = <1,y> = r < rhs, s = -t; fix entries that leave the
  // support of x or of y                                        (:74-113)
  int cx; R sx; int cy; R sy;
  row_count_sum_gt<R>(ra, cut_x, cx, sx);
  row_count_sum_gt<R>(rb, cut_y, cy, sy);
  int mm = cx + cy;
  const int it_max = mm + 2;
  t = (sx - sy) / static_cast<R>(mm);
  for (int it = 0;; ++it) {
    R sum_x = 0, sum_y = 0; int n_x = 0, n_y = 0;
    ra.for_each([&](typename RowA::data_type xd, int) {
      R x = static_cast<R>(xd);
      if (x > cut_x && !(x > t)) { sum_x += x; ++n_x; }
    });
    rb.for_each([&](typename RowB::data_type yd, int) {
      R y = static_cast<R>(yd);
      if (y > cut_y && !(y > -t)) { sum_y += y; ++n_y; }
    });
    sum_x = warp_sum(sum_x); sum_y = warp_sum(sum_y);
    n_x = warp_sum(n_x); n_y = warp_sum(n_y);
    const R infeas = sum_x - sum_y - static_cast<R>(n_x + n_y) * t;
    R tt;
    if (n_y > 0 && infeas > eps && it <= it_max) {
      cut_y = max_(cut_y, -t);
      tt = static_cast<R>(mm) * t + sum_y;
      mm -= n_y; cy -= n_y;
    } else if (n_x > 0 && infeas < -eps && it <= it_max) {
      cut_x = max_(cut_x, t);
      tt = static_cast<R>(mm) * t - sum_x;
      mm -= n_x; cx -= n_x;
    } else {
      cut_x = max_(cut_x, t); cut_y = max_(cut_y, -t);
      cx -= n_x; cy -= n_y;
      break;
    }
    if (mm > 0) t = tt / static_cast<R>(mm); else break;
  }
  out.a = make_thr(t, lo, hi, 0, cx, num<R>::inf(), cut_x);
  out.b = make_thr(-t, lo, hi, 0, cy, num<R>::inf(), cut_y);
  return out;
}

}  // namespace sdcab
