// Register-resident rows: one warp keeps a whole row in registers (16-byte
// vector loads, NV vectors per lane), so the matrix is read from HBM exactly
// once and written exactly once, and every pass of a threshold search runs out
// of the register file.
//
// On top of that, the top-k operators shrink the row before searching: only
// entries above a cut that provably contains the support take part, and those
// (a dozen for Gaussian rows of length 1000) are compacted to one entry per
// lane, where every reduction is a handful of shuffles.  Rows whose candidates
// do not fit 32 lanes, or that need the general cone search, run the same
// threshold code on the full register row instead.
#pragma once

#include <type_traits>

#include "common_host.h"
#include "prox_core.cuh"

namespace sdcab {

constexpr int kNoFastPath = 1;
constexpr int kFastThreads = 128;
// Resident blocks per SM the register allocation aims for.  Operators that keep
// the row in registers through their search: double thresholds need more live
// registers, and spilling them costs more than the lost warps.  The top-k
// projections read the row a second time for the final map instead (see the
// kernel), so their search runs in 64-72 registers and eight (seven for the
// simplex with double thresholds) blocks fit; measured fastest at these values.
// The knapsack family (knapsack_eq / _le / _le_biased) does the same once a lane holds four
// vectors or more; with two vectors per lane (config 1's 100 doubles) keeping the row was
// measured faster.
template <int PROX, int NV> struct KnapsackStaged {
  static constexpr bool value = (PROX == kKnapsackEq || PROX == kKnapsackLe || PROX == kKnapsackLeBiased) &&
                                NV >= 4;
};
template <typename Data, typename R, int PROX, int NV> struct FastMinBlocks {
  static constexpr bool kTopk = (PROX == kTopkSimplex || PROX == kTopkSimplexBiased ||
                                 PROX == kTopkCone || PROX == kTopkConeBiased);
  static constexpr bool kSimplex = (PROX == kTopkSimplex || PROX == kTopkSimplexBiased);
  static constexpr bool kDouble = sizeof(R) == 8;
  static constexpr bool kEntropic = sizeof(Data) == 4 && (PROX == kTopkEntropy || PROX == kEntropy);
  static constexpr bool kKnapStaged = KnapsackStaged<PROX, NV>::value;
  // the simplex projection of short rows (config 1's 100 doubles) fits eight blocks as well
  static constexpr bool kShortSimplex = (PROX == kKnapsackEq) && NV == 2;
  static constexpr int value = kTopk ? ((kDouble && kSimplex) ? 7 : 8)
                                     : ((kEntropic || kKnapStaged || kShortSimplex || PROX == kTwoSimplex)
                                            ? 8 : (kDouble ? 5 : 6));
};

template <typename Data> struct VecOf;
template <> struct VecOf<float> { typedef float4 type; static constexpr int N = 4; };
template <> struct VecOf<double> { typedef double2 type; static constexpr int N = 2; };

// A row held in registers: lane l owns vectors l, 32 + l, 64 + l, ...
template <typename Data, int NV>
struct RegRow {
  typedef Data data_type;
  typedef typename VecOf<Data>::type Vec;
  static constexpr int VN = VecOf<Data>::N;
  Vec v[NV];
  int m;

  __device__ __forceinline__ int size() const { return m; }

  __device__ __forceinline__ void load(const Data* __restrict__ g, int lane) {
    const Vec* gv = reinterpret_cast<const Vec*>(g);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int vi = j * 32 + lane;
      if (vi * VN < m) {
        v[j] = __ldcs(gv + vi);
      } else {
        Data* e = reinterpret_cast<Data*>(&v[j]);
#pragma unroll
        for (int c = 0; c < VN; ++c) e[c] = -num<Data>::inf();
      }
    }
  }

  // First of two reads of a row: cached in L2 (not L1), so that the second read --
  // after the search, when the row's registers have been given up -- finds it there.
  __device__ __forceinline__ void load_keep(const Data* __restrict__ g, int lane) {
    const Vec* gv = reinterpret_cast<const Vec*>(g);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int vi = j * 32 + lane;
      if (vi * VN < m) {
        v[j] = __ldcg(gv + vi);
      } else {
        Data* e = reinterpret_cast<Data*>(&v[j]);
#pragma unroll
        for (int c = 0; c < VN; ++c) e[c] = -num<Data>::inf();
      }
    }
  }

  template <typename F>
  __device__ __forceinline__ void for_each(F&& f) const {
    const int lane = static_cast<int>(threadIdx.x) & 31;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int base = (j * 32 + lane) * VN;
      if (base < m) {
        const Data* e = reinterpret_cast<const Data*>(&v[j]);
#pragma unroll
        for (int c = 0; c < VN; ++c) f(e[c], base + c);
      }
    }
  }

  // like store, the map also gets the entry's index
  template <typename F>
  __device__ __forceinline__ void store_indexed(Data* __restrict__ g, int lane, F&& f) const {
    Vec* gv = reinterpret_cast<Vec*>(g);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int vi = j * 32 + lane;
      if (vi * VN < m) {
        Vec o = v[j];
        Data* e = reinterpret_cast<Data*>(&o);
#pragma unroll
        for (int c = 0; c < VN; ++c) e[c] = f(e[c], vi * VN + c);
        __stcs(gv + vi, o);
      }
    }
  }

  template <typename F>
  __device__ __forceinline__ void store(Data* __restrict__ g, int lane, F&& f) const {
    Vec* gv = reinterpret_cast<Vec*>(g);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int vi = j * 32 + lane;
      if (vi * VN < m) {
        Vec o = v[j];
        Data* e = reinterpret_cast<Data*>(&o);
#pragma unroll
        for (int c = 0; c < VN; ++c) e[c] = f(e[c]);
        __stcs(gv + vi, o);
      }
    }
  }
};

// At most one entry per lane (the compacted candidates); `reported` is what
// size() answers, which the caller sets to the true row length where the
// algorithm asks "is this the whole row?".
template <typename Data>
struct LaneRow {
  typedef Data data_type;
  Data x;
  bool valid;
  int reported;
  __device__ __forceinline__ int size() const { return reported; }
  template <typename F>
  __device__ __forceinline__ void for_each(F&& f) const {
    if (valid) f(x, static_cast<int>(threadIdx.x) & 31);
  }
};

// Descending bitonic sort of one value per lane.
template <typename T>
__device__ __forceinline__ T warp_sort_desc(T v, int lane) {
#pragma unroll
  for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      const T w = __shfl_xor_sync(kFullMask, v, j);
      const bool upper = (lane & j) != 0;          // partner has the smaller lane id
      const bool desc = (lane & k) == 0 || k == 32;  // direction of this block
      const bool keep_max = (upper != desc);
      v = keep_max ? (w > v ? w : v) : (w < v ? w : v);
    }
  }
  return v;
}

// Warp-wide maximum in one instruction (redux.sync on sm_100a handles f32;
// doubles take the shuffle butterfly).
__device__ __forceinline__ float warp_max_fast(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ double warp_max_fast(double v) { return warp_max(v); }

// The (k+1)-th largest of the 32 lane values (k <= 31), counting repeats:
// repeatedly take the warp maximum and retire the lanes that hold it.
template <typename T>
__device__ __forceinline__ T kth_largest_of_lanes(T v, int k, int lane) {
  (void)lane;
  int seen = 0;
  T cur = v, top = -num<T>::inf();
  for (int round = 0; round <= k; ++round) {
    top = warp_max_fast(cur);
    const unsigned hit = __ballot_sync(kFullMask, cur == top);
    seen += __popc(hit);
    if (seen > k || top == -num<T>::inf()) break;
    cur = (cur == top) ? -num<T>::inf() : cur;
  }
  return top;
}

// The cut below which no entry can belong to the support, from the lane maxima:
// tau = (k+1)-th largest lane maximum is a lower bound of the (k+1)-th largest
// entry of the row.
template <typename Data, int NV>
__device__ __forceinline__ Data lane_max_cut(const RegRow<Data, NV>& row, int k, int lane) {
  // balanced tree: short dependency chains
  Data vm[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const Data* e = reinterpret_cast<const Data*>(&row.v[j]);
    Data a = e[0];
#pragma unroll
    for (int c = 1; c < RegRow<Data, NV>::VN; ++c) a = max_(a, e[c]);
    if (RegRow<Data, NV>::VN == 4) a = max_(max_(e[0], e[1]), max_(e[2], e[3]));
    vm[j] = a;
  }
#pragma unroll
  for (int w = 1; w < NV; w <<= 1) {
#pragma unroll
    for (int j = 0; j + w < NV; j += 2 * w) vm[j] = max_(vm[j], vm[j + w]);
  }
  const Data lm = vm[0];
  return kth_largest_of_lanes(lm, k, lane);
}

// Compacts the entries with x > cut to one per lane through shared memory;
// slots are handed out by a shared-memory counter (the order is irrelevant, the
// candidates are sorted afterwards).  Returns their number; the LaneRow is only
// valid if that number is <= 32.  *counter must be 0 on entry and is left at 0.
template <typename Data, int NV>
__device__ __forceinline__ int compact_candidates(const RegRow<Data, NV>& row, Data cut,
                                                  Data* __restrict__ slots, int* counter,
                                                  int lane, LaneRow<Data>& out) {
  row.for_each([&](Data x, int) {
    if (x > cut) {
      const int pos = atomicAdd(counter, 1);
      if (pos < 32) slots[pos] = x;
    }
  });
  __syncwarp();
  const int total = *counter;
  out.valid = lane < total;
  out.x = (lane < total && total <= 32) ? slots[lane] : -num<Data>::inf();
  __syncwarp();
  if (lane == 0) *counter = 0;
  __syncwarp();
  return total;
}

// Largest float/double not above a Result value (so that Data-precision
// comparisons against it are equivalent to Result-precision ones).
__device__ __forceinline__ float round_down(double v, float) { return __double2float_rd(v); }
__device__ __forceinline__ float round_down(float v, float) { return v; }
__device__ __forceinline__ double round_down(double v, double) { return v; }
__device__ __forceinline__ double round_down(float v, double) { return static_cast<double>(v); }

// 1 / j for the set sizes that occur among at most 32 candidates: the searches
// divide by small counts, and a multiplication by the tabulated reciprocal (one
// rounding more than the division, far inside every tolerance) is a single
// instruction where the division is a routine of thirty.
static __constant__ double kReciprocal[33] = {
    0.0, 1.0, 1.0 / 2, 1.0 / 3, 1.0 / 4, 1.0 / 5, 1.0 / 6, 1.0 / 7, 1.0 / 8, 1.0 / 9, 1.0 / 10,
    1.0 / 11, 1.0 / 12, 1.0 / 13, 1.0 / 14, 1.0 / 15, 1.0 / 16, 1.0 / 17, 1.0 / 18, 1.0 / 19, 1.0 / 20,
    1.0 / 21, 1.0 / 22, 1.0 / 23, 1.0 / 24, 1.0 / 25, 1.0 / 26, 1.0 / 27, 1.0 / 28, 1.0 / 29, 1.0 / 30,
    1.0 / 31, 1.0 / 32};
template <typename R>
__device__ __forceinline__ R over_count(R x, int j) { return x * static_cast<R>(kReciprocal[j]); }

// ---- the compacted candidates, sorted ---------------------------------------
// Lane i holds the i-th largest candidate (lanes >= n hold -inf) and the sum
// of the first i + 1 of them, so a sum or a count over any value range is one
// ballot plus one or two shuffles.
template <typename R>
struct Sorted {
  R s, P;
  int n;
  const R* shared;   // optional copy in shared memory: 32 values, then 32 prefix sums
  __device__ __forceinline__ R at(int i) const {
    return shared ? shared[i] : __shfl_sync(kFullMask, s, i);
  }
  // sum of the i largest candidates
  __device__ __forceinline__ R pre(int i) const {
    if (shared) return i > 0 ? shared[32 + i - 1] : R(0);
    const R v = __shfl_sync(kFullMask, P, i > 0 ? i - 1 : 0);
    return i > 0 ? v : R(0);
  }
  __device__ __forceinline__ int count_gt(R c) const {
    return __popc(__ballot_sync(kFullMask, s > c));
  }
};

// `shared` (64 entries of this warp, optional) receives the sorted values and their
// prefix sums, which turns every later look-up by index into one broadcast load.
template <typename R, typename Data>
__device__ __forceinline__ Sorted<R> sort_candidates(const LaneRow<Data>& cand, int n, int lane,
                                                     R* shared = nullptr) {
  Sorted<R> out;
  out.shared = shared;
  const Data v = warp_sort_desc(cand.x, lane);
  out.s = static_cast<R>(v);
  out.n = n;
  R p = (lane < n) ? out.s : R(0);
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const R up = __shfl_up_sync(kFullMask, p, o);
    if (lane >= o) p += up;
  }
  out.P = p;
  if (shared) {
    __syncwarp();   // earlier readers of the previous row's copy are done
    shared[lane] = out.s;
    shared[32 + lane] = p;
    __syncwarp();
  }
  return out;
}

// Zero / constant / general classification on sorted candidates
// (include/sdca/prox/topk_cone.h:18-55 of the reference); `m` is the length of
// the whole row.  Needs more than k candidates.
template <typename R>
__device__ __forceinline__ Projection sorted_special_cases(const Sorted<R>& c, int m, int k,
                                                           R inv_div, Thr<R>& thr) {
  const R eps = 16 * num<R>::eps();
  const R sum_k = c.pre(k);
  if (sum_k <= eps) {
    thr = make_thr(R(0), R(0), R(0), 0, 0, num<R>::inf(), num<R>::inf());
    return kProjZero;
  }
  const R v_k = c.at(k - 1);
  const R hi = sum_k * inv_div;
  const R t = v_k - hi;
  if (k == m || t >= c.at(k) - eps) {
    thr = make_thr(t, R(0), hi, k, 0, v_k, v_k);
    return kProjConstant;
  }
  return kProjGeneral;
}

// Variable fixing for  <1,x> = rhs, 0 <= x <= hi  on sorted candidates: the
// iteration of thr_knapsack_eq with the free entries kept as the index range
// [f0, f1) of the sorted order.  Entries that are not candidates are below
// every threshold the iteration can reach and contribute lo = 0.
template <typename R>
__device__ __forceinline__ Thr<R> sorted_knapsack_eq(const Sorted<R>& c, R hi, R rhs, R& sum_U) {
  const int n = c.n;
  const R eps = num<R>::eps() * max_(R(1), abs_(rhs));
  int f0 = 0, f1 = n, mfree = n;
  R S0 = 0, S1 = c.pre(n);
  R t = (S1 - rhs) / static_cast<R>(n);
  for (int it = 0;; ++it) {
    const R thi = hi + t;
    int a = c.count_gt(t);
    a = min(max(a, f0), f1);           // lo-set: [a, f1)
    int b = min(c.count_gt(thi), a);
    b = max(b, f0);                    // hi-set: [f0, b)
    const R Pa = c.pre(a), Pb = c.pre(b);
    const int n_lo = f1 - a, n_hi = b - f0;
    const R sum_lo = S1 - Pa, sum_hi = Pb - S0;
    const R s_hi = static_cast<R>(n_hi) * hi;
    const R infeas = sum_hi + sum_lo - s_hi - static_cast<R>(n_hi + n_lo) * t;
    R tt;
    if (n_hi > 0 && infeas > eps && it <= n) {
      tt = static_cast<R>(mfree) * t - sum_hi + s_hi;
      mfree -= n_hi; f0 = b; S0 = Pb;
    } else if (n_lo > 0 && infeas < -eps && it <= n) {
      tt = static_cast<R>(mfree) * t - sum_lo;
      mfree -= n_lo; f1 = a; S1 = Pa;
    } else {
      sum_U = Pb;
      return make_thr(t, R(0), hi, b, a - b, min_(thi, b > 0 ? c.at(b - 1) : num<R>::inf()), t);
    }
    if (mfree > 0) {
      t = tt / static_cast<R>(mfree);
    } else {
      sum_U = S0;
      return make_thr(t, R(0), hi, f0, 0, thi, thi);
    }
  }
}

// Direct solution of  <1,x> = rhs, 0 <= x <= hi = rhs/k  on sorted candidates.
// With the u largest entries at hi, the others solve an ordinary simplex
// projection onto the remaining mass rhs - u*hi, whose threshold over sorted
// data is tau_j = (sum of the first j of them - mass) / j for the largest j with
// s_j > tau_j.  The pair (u, tau) is the solution when it is consistent (entry u
// not above hi, entry u-1 above it), and the smallest consistent u is the unique
// KKT point that the reference's variable fixing converges to
// (include/sdca/prox/knapsack_eq.h:25-109).  Lane u works out its own candidate:
// the sorted values and prefix sums go to shared memory once and every lane walks
// over them, so all u <= k are tried in one pass instead of one round each.
// `sorted` holds 2 x 32 entries of this warp.
template <typename R>
__device__ __forceinline__ bool sorted_capped_simplex(const Sorted<R>& c, R hi, R rhs, int k,
                                                      int lane, R* sorted, Thr<R>& thr, R& sum_U) {
  const int n = c.n;
  const R inf = num<R>::inf();
  R* sm_s = sorted;
  R* sm_P = sorted + 32;
  sm_s[lane] = c.s;
  sm_P[lane] = c.P;
  __syncwarp();
  const int u = lane;
  const bool live = (u <= k) && (u < n);
  const R Pu = (u > 0) ? sm_P[(u - 1) & 31] : R(0);
  const R s_um1 = (u > 0) ? sm_s[(u - 1) & 31] : inf;
  // s_j > tau_j  <=>  (j - u + 1) * s_j > P_j - (P_u + mass): no division until j is known
  const R base = Pu + (rhs - static_cast<R>(u) * hi);
  // The entries above their tau_j form a prefix of u, u + 1, ..., so the last one is
  // found by bisection: five probes cover 32 candidates.
  int last = -1;
  {
    int lo_j = u, hi_j = n;          // the last j that passes lies in [lo_j - 1, hi_j)
#pragma unroll
    for (int step = 0; step < 5; ++step) {
      const int mid = (lo_j + hi_j) >> 1;
      const bool probe = lo_j < hi_j;
      const int jj = probe ? mid : 0;
      const R sj = sm_s[jj], Pj = sm_P[jj];
      const bool ok = probe && (sj * static_cast<R>(jj - u + 1) > Pj - base);
      lo_j = ok ? mid + 1 : lo_j;
      hi_j = (probe && !ok) ? mid : hi_j;
    }
    last = lo_j - 1;
    if (last < u) last = -1;
  }
  R t;
  int inside;
  bool consistent;
  if (last < 0) {
    // nothing strictly inside: the u capped entries carry all the mass
    t = s_um1 - hi;
    inside = 0;
    consistent = (u > 0) && (c.s <= t);
  } else {
    inside = last - u + 1;
    t = over_count(sm_P[last] - base, inside);
    consistent = (c.s - t <= hi) && (u == 0 || s_um1 - t > hi);
  }
  __syncwarp();
  const unsigned found = __ballot_sync(kFullMask, live && consistent);
  if (found == 0u) return false;
  const int w = __ffs(found) - 1;
  const R t_w = __shfl_sync(kFullMask, t, w);
  const R prev_w = __shfl_sync(kFullMask, s_um1, w);
  const int inside_w = __shfl_sync(kFullMask, inside, w);
  sum_U = __shfl_sync(kFullMask, Pu, w);
  thr = make_thr(t_w, R(0), hi, w, inside_w, prev_w, inside_w > 0 ? t_w : prev_w);
  return true;
}

enum FastStatus { kFastDone = 0, kFastNeedsFullRow = 1 };

// Constants of the top-k operators that do not depend on the row; worked out
// once per thread, outside the loop over rows (three of them are divisions).
template <typename R>
struct TopkConsts {
  R K, H, rho_k2, inv_div, inv_K, eps_rhs;
  __device__ __forceinline__ TopkConsts(int k, R rhs, R rho) {
    K = static_cast<R>(k);
    H = rhs / K;
    rho_k2 = rho * K * K;
    inv_div = R(1) / (K + rho_k2);
    inv_K = R(1) / K;
    eps_rhs = num<R>::eps() * max_(R(1), abs_(rhs));
  }
};

// Top-k simplex (rho = 0) and its biased form.  Returns kFastNeedsFullRow when
// the row has to go through the general search on the full row.
template <typename R, typename Data, int NV>
__device__ __forceinline__ FastStatus fast_topk_simplex(const RegRow<Data, NV>& row, int k, R rhs,
                                                        R rho, const TopkConsts<R>& tc, Data* slots,
                                                        int* counter, R* sorted, int lane,
                                                        Thr<R>& thr) {
  const int m = row.size();
  if (k > 31 || m <= 32) return kFastNeedsFullRow;
  const R K = tc.K, H = tc.H;
  const Data tau = lane_max_cut(row, k, lane);
  // support of the knapsack step: a_i > t >= v_(k+1) - rhs/k >= tau - rhs/k
  const Data cut = round_down(static_cast<R>(tau) - H - abs_(static_cast<R>(tau)) * num<R>::eps() * 4,
                              Data(0));
  LaneRow<Data> cand;
  const int total = compact_candidates(row, cut, slots, counter, lane, cand);
  if (total > 32 || total <= k) return kFastNeedsFullRow;
  const Sorted<R> c = sort_candidates<R>(cand, total, lane);
  const R eps = tc.eps_rhs;
  const R rho_k2 = tc.rho_k2;
  const Projection proj = sorted_special_cases<R>(c, m, k, tc.inv_div, thr);
  if (proj == kProjZero) return kFastDone;
  R sum_U;
  if (proj == kProjConstant) {
    if (K * thr.hi > rhs + eps) {
      if (!sorted_capped_simplex<R>(c, H, rhs, k, lane, sorted, thr, sum_U))
        thr = sorted_knapsack_eq<R>(c, H, rhs, sum_U);
    }
    return kFastDone;
  }
  if (!sorted_capped_simplex<R>(c, H, rhs, k, lane, sorted, thr, sum_U))
    thr = sorted_knapsack_eq<R>(c, H, rhs, sum_U);
  bool lt;
  if (thr.nU == 0) {
    lt = thr.t < rho * rhs - eps;
  } else {
    const R num_U = static_cast<R>(thr.nU);
    lt = K * (sum_U + (K - num_U) * thr.t) < rhs * (num_U + rho_k2) - eps;
  }
  return lt ? kFastNeedsFullRow : kFastDone;
}

// Top-k cone.  For rho = 0 the first candidate of the search (U empty) has
// t = 0 and M = {a > 0}: one pass for the sum of the positive entries decides
// it; anything else takes the general search.
template <typename R, typename Data, int NV>
__device__ __forceinline__ FastStatus fast_topk_cone(const RegRow<Data, NV>& row, int k, R rho,
                                                     const TopkConsts<R>& tc, Data* slots, int* counter,
                                                     R* sorted, int lane, Thr<R>& thr) {
  const int m = row.size();
  if (k > 31 || m <= 32 || rho != 0) return kFastNeedsFullRow;
  const R K = tc.K;
  const Data tau = lane_max_cut(row, k, lane);
  const Data cut = round_down(static_cast<R>(tau) - abs_(static_cast<R>(tau)) * num<R>::eps() * 4
                              - num<R>::tiny(), Data(0));
  LaneRow<Data> cand;
  const int total = compact_candidates(row, cut, slots, counter, lane, cand);
  if (total > 32 || total <= k) return kFastNeedsFullRow;
  const R inv_K = tc.inv_K;
  const R eps = 16 * num<R>::eps();
  // sum and count of the positive entries, taken now so that the row's registers
  // are free during the search.  U is empty on the branch that uses them, so no
  // output attains hi and only the acceptance test below depends on the sum:
  // float data is summed per lane in float (four chains), across lanes in R,
  // and a test that is not clear-cut is left to the general search.
  int j = 0; R s = 0;
  constexpr bool kFloatSums = std::is_same<Data, float>::value && std::is_same<R, double>::value;
  if (kFloatSums) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    int cnt[4] = {0, 0, 0, 0};
#pragma unroll
    for (int jv = 0; jv < NV; ++jv) {
      // vectors past the end of the row hold -inf and add nothing
      const float* e = reinterpret_cast<const float*>(&row.v[jv]);
#pragma unroll
      for (int cc = 0; cc < RegRow<Data, NV>::VN; ++cc) {
        acc[cc & 3] += fmaxf(e[cc], 0.0f);
        cnt[cc & 3] += (e[cc] > 0.0f) ? 1 : 0;
      }
    }
    j = warp_sum((cnt[0] + cnt[1]) + (cnt[2] + cnt[3]));
    s = warp_sum((static_cast<R>(acc[0]) + static_cast<R>(acc[1])) +
                 (static_cast<R>(acc[2]) + static_cast<R>(acc[3])));
  } else {
    row.for_each([&](Data xd, int) {
      if (xd > Data(0)) { ++j; s += static_cast<R>(xd); }
    });
    j = warp_sum(j); s = warp_sum(s);
  }
  const Sorted<R> c = sort_candidates<R>(cand, total, lane);
  if (sorted_special_cases<R>(c, m, k, inv_K, thr) != kProjGeneral) return kFastDone;
  bool clear_cut = true;
  if (kFloatSums) {
    const R hi_est = s * inv_K;
    const R mx = c.at(0);
    clear_cut = abs_(mx - hi_est) > R(1e-4) * max_(abs_(hi_est), abs_(mx));
  }
  if (!clear_cut) return kFastNeedsFullRow;
  // U empty: t = 0 and hi = K s / K^2 = s / K (include/sdca/prox/topk_cone.h:83-98)
  const R t = R(0);
  const R hi = s * inv_K;
  if (j > 0 && c.at(0) - eps <= hi + t) {
    thr = make_thr(t, R(0), hi, 0, j, num<R>::inf(), t);
    return kFastDone;
  }
  return kFastNeedsFullRow;
}

// Top-k cone with rho > 0 (include/sdca/prox/topk_cone_biased.h:8-113).  For a set U of the
// u largest entries the pair (M, t) is the root of
//     F_u(t) = up * sum_{i not in U} (a_i - t)_+  -  (k - u)^2 t  -  (k - u) sum_U,   up = u + rho k^2,
// decreasing in t, and the search accepts the first u whose (t, hi) passes the reference's
// inequalities.  With rho > 0 every root is well above the bulk of the row, so the search
// needs only the entries above a cut below all the roots.  Such a cut comes from a few
// entries of the row: with v_1 >= v_2 >= ... the J largest lane maxima (each an entry of its
// own), at most u of them lie in U and sum_U <= u v_1, hence
//     F_u(t) >= up * sum_{i = u+1..J} (v_i - t)_+  -  (k - u)^2 t  -  (k - u) u v_1,
// whose root L_u bounds the root of F_u from below; lane u solves its own L_u.  The entries
// above min_u L_u (and at least the k + 1 largest) are compacted and sorted, and lane u then
// runs the Newton iteration of the general routine on the sorted candidates -- a count and a
// prefix-sum look-up per step instead of a pass over the row -- followed by the acceptance
// test; the smallest u that passes wins, as in the sequential search.
template <typename R, typename Data, int NV>
__device__ __forceinline__ FastStatus fast_topk_cone_biased(const RegRow<Data, NV>& row, int k, R rho,
                                                            const TopkConsts<R>& tc, Data* slots,
                                                            int* counter, R* sorted, int lane,
                                                            Thr<R>& thr) {
  const int m = row.size();
  if (k > 8 || m <= 32 || !(rho > 0)) return kFastNeedsFullRow;
  const R K = tc.K, rho_k2 = tc.rho_k2;
  const R eps = 16 * num<R>::eps();
  const int J = k + 4;
  // the J largest lane maxima, in descending order, into shared memory
  {
    Data lmd = -num<Data>::inf();
    row.for_each([&](Data x, int) { lmd = max_(lmd, x); });
    float cur = round_down(lmd, float());
    float top = warp_max_fast(cur);
    if (!(top > -num<float>::inf())) return kFastNeedsFullRow;
    for (int j = 0; j < J; ++j) {
      if (lane == 0) sorted[j] = static_cast<R>(top);
      const unsigned hit = __ballot_sync(kFullMask, cur == top);
      if (lane == __ffs(hit) - 1) cur = -num<float>::inf();
      top = warp_max_fast(cur);
    }
    __syncwarp();
  }
  // lane u < k: the root L_u of the lower bound of F_u
  R bound = num<R>::inf();
  const R v1 = sorted[0];
  if (lane < k) {
    const int u = lane;
    const R kmu = K - static_cast<R>(u), up = static_cast<R>(u) + rho_k2;
    const R fixed = kmu * static_cast<R>(u) * v1;
    int cnt = 0; R sum = 0;
    for (int i = u; i < J; ++i) {
      const R v = sorted[i];
      if (v > -num<R>::inf()) { ++cnt; sum += v; }
    }
    R t = (up * sum - fixed) / (kmu * kmu + up * static_cast<R>(cnt));
    // the values above t are a prefix of v_{u+1}, v_{u+2}, ...: drop from the end
    while (cnt > 0 && !(sorted[u + cnt - 1] > t)) {
      sum -= sorted[u + cnt - 1];
      --cnt;
      t = (up * sum - fixed) / (kmu * kmu + up * static_cast<R>(cnt));
    }
    bound = t;
  }
  // the k + 1 largest entries have to be candidates as well
  if (lane == k) bound = sorted[k];
  bound = warp_min(bound);
  __syncwarp();
  if (!(bound > -num<R>::inf())) return kFastNeedsFullRow;
  const Data cut = round_down(bound - (abs_(bound) + abs_(v1) + R(1)) * eps, Data());
  LaneRow<Data> cand;
  const int total = compact_candidates(row, cut, slots, counter, lane, cand);
  if (total > 32 || total <= k) return kFastNeedsFullRow;
  const Sorted<R> c = sort_candidates<R>(cand, total, lane);
  if (sorted_special_cases<R>(c, m, k, tc.inv_div, thr) != kProjGeneral) return kFastDone;
  R* sm_s = sorted;
  R* sm_P = sorted + 32;
  sm_s[lane] = c.s;
  sm_P[lane] = c.P;
  __syncwarp();
  const int n = total;
  bool pass = false;
  R t_u = 0, hi_u = 0, minU_u = num<R>::inf();
  int j_u = 0;
  if (lane <= k) {
    const int u = lane;
    const R kmu = K - static_cast<R>(u), up = static_cast<R>(u) + rho_k2;
    const R sum_U = (u > 0) ? sm_P[u - 1] : R(0);
    const R min_U = (u > 0) ? sm_s[u - 1] : num<R>::inf();
    const R s_u = sm_s[u];                 // the largest entry outside U (n > k >= u)
    int j; R sum_M;
    bool valid = true;
    if (u == k) {
      if (up > 0) { j = 1; sum_M = s_u; } else { j = 0; sum_M = 0; valid = false; }
    } else {
      // Newton steps from the left, starting on the piece of the cut
      j = n - u; sum_M = sm_P[n - 1] - sum_U;
      for (int it = 0; it <= 32; ++it) {
        const R D = kmu * kmu + up * static_cast<R>(j);
        const R t = (up * sum_M - kmu * sum_U) / D;
        // candidates outside U that exceed t: a prefix of s_u, s_{u+1}, ...
        int g = u;
        while (g < n && sm_s[g] > t) ++g;
        const int cj = g - u;
        if (cj == j) break;
        j = cj;
        sum_M = (g > 0 ? sm_P[g - 1] : R(0)) - sum_U;
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
        else if (j == 0) ok = (s_u - eps <= t);
        pass = ok;
      }
      t_u = t; hi_u = hi; minU_u = min_U; j_u = j;
    }
  }
  __syncwarp();
  const unsigned found = __ballot_sync(kFullMask, pass);
  if (found == 0u) return kFastNeedsFullRow;
  const int w = __ffs(found) - 1;
  const R t = __shfl_sync(kFullMask, t_u, w);
  const R hi = __shfl_sync(kFullMask, hi_u, w);
  const R min_U = __shfl_sync(kFullMask, minU_u, w);
  const int j = __shfl_sync(kFullMask, j_u, w);
  // all of M has to be among the candidates: the cut lies below every root by construction,
  // and a root that reaches down to the cut is left to the general search
  if (!(t > static_cast<R>(cut))) return kFastNeedsFullRow;
  thr = make_thr(t, R(0), hi, w, j, min_U, (j > 0) ? t : min_U);
  return kFastDone;
}

// ---- knapsack with lo = 0 (the simplex of include/sdca/prox/knapsack_eq.h) -----
// When no entry reaches the upper bound, the solution has t >= max - rhs (the
// largest entry alone contributes max - t <= rhs), so the support lies among the
// entries above max - rhs: a handful for rows whose entries are not bunched at
// the top.  Those are compacted to one per lane; every lane ranks its entry
// among the candidates and sums the candidates ranked before it in one pass of
// broadcasts (no sort), which gives the threshold of every possible support
// size at once: t_j = (sum of the j largest - rhs) / j, and the support is the
// largest j whose j-th largest entry exceeds t_j.  The reference reaches the
// same t by Kiwiel's variable fixing, several dependent reductions over the row.
template <typename R, typename Data, int NV>
__device__ __forceinline__ FastStatus fast_knapsack_eq(const RegRow<Data, NV>& row, R hi, R rhs,
                                                       Data* slots, int* counter, int lane,
                                                       Thr<R>& thr) {
  Data lm = -num<Data>::inf();
  row.for_each([&](Data x, int) { lm = max_(lm, x); });
  // a lower bound of the maximum through the one-instruction float reduction
  float cur = round_down(lm, float());
  const float below = warp_max_fast(cur);
  if (!(below > -num<float>::inf())) return kFastNeedsFullRow;
  const R below_r = static_cast<R>(below);
  // t is the largest of the t_j, and any j entries of the row bound the sum of its j largest
  // from below: the largest lane maxima (each an entry of its own) give t >= (their sum - rhs) / j.
  // For long rows that cut is far tighter than max - rhs (N(0,1), m = 1000: about 4 candidates
  // instead of 30, which would overflow the 32 slots on a quarter of the rows).
  R bound = below_r - rhs;
  if (NV >= 4) {
    R sum = below_r;
    float top = below;
#pragma unroll
    for (int j = 2; j <= 4; ++j) {
      const unsigned hit = __ballot_sync(kFullMask, cur == top);
      if (lane == __ffs(hit) - 1) cur = -num<float>::inf();
      top = warp_max_fast(cur);
      if (!(top > -num<float>::inf())) break;
      sum += static_cast<R>(top);
      bound = max_(bound, over_count(sum - rhs, j));
    }
  }
  const Data cut = round_down(bound - (abs_(below_r) + rhs) * num<R>::eps() * 8, Data());
  LaneRow<Data> cand;
  const int total = compact_candidates(row, cut, slots, counter, lane, cand);
  if (total > 32 || total < 1) return kFastNeedsFullRow;
  const bool mine = lane < total;
  const R v = static_cast<R>(cand.x);
  int rank = 0;
  R before = 0;                       // sum of the candidates ranked before this one
  for (int j = 0; j < total; ++j) {
    const R vj = __shfl_sync(kFullMask, v, j);
    const bool first = (vj > v) || (vj == v && j < lane);
    rank += first ? 1 : 0;
    before += first ? vj : R(0);
  }
  const R t_mine = over_count(before + v - rhs, rank + 1);
  const bool inside = mine && v > t_mine;
  int size = inside ? rank + 1 : 0;
  size = __reduce_max_sync(kFullMask, size);
  if (size < 1) return kFastNeedsFullRow;
  const unsigned who = __ballot_sync(kFullMask, mine && rank == size - 1);
  const R t = __shfl_sync(kFullMask, t_mine, __ffs(who) - 1);
  // an entry at the upper bound: the general routine fixes it first
  if (__any_sync(kFullMask, mine && v - t > hi)) return kFastNeedsFullRow;
  thr = make_thr(t, R(0), hi, 0, size, hi + t, t);
  return kFastDone;
}

// knapsack_le with lo = 0 (include/sdca/prox/knapsack_le.h:17-44): the sum of the row clipped
// to [0, hi] decides between t = 0 and the equality-constrained projection.
template <typename R, typename Data, int NV>
__device__ __forceinline__ FastStatus fast_knapsack_le(const RegRow<Data, NV>& row, R hi, R rhs,
                                                       Data* slots, int* counter, int lane,
                                                       Thr<R>& thr) {
  const R eps = num<R>::eps() * max_(R(1), abs_(rhs));
  int n_hi = 0, n_mid = 0;
  R sum_mid = 0;
  constexpr bool kFloatSums = std::is_same<Data, float>::value && std::is_same<R, double>::value;
  if (kFloatSums) {
    // Float data, double thresholds: the sum of the row clipped to [0, hi] only decides which
    // branch is taken, so it is formed per lane in float (four chains, hi rounded to float)
    // and across lanes in R; a sum within 1e-4 of rhs is not clear-cut and is left to the
    // general routine.  The set sizes are not counted here: this path only feeds the map
    // x -> clip(x - t, 0, hi), which does not use them.
    const float hif = static_cast<float>(hi);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int jv = 0; jv < NV; ++jv) {
      const float* e = reinterpret_cast<const float*>(&row.v[jv]);   // padding holds -inf
#pragma unroll
      for (int cc = 0; cc < RegRow<Data, NV>::VN; ++cc)
        acc[cc & 3] += fminf(fmaxf(static_cast<float>(e[cc]), 0.0f), hif);
    }
    const R s_est = warp_sum((static_cast<R>(acc[0]) + static_cast<R>(acc[1])) +
                             (static_cast<R>(acc[2]) + static_cast<R>(acc[3])));
    if (!(abs_(s_est - rhs) > R(1e-4) * max_(abs_(s_est), abs_(rhs)))) return kFastNeedsFullRow;
    if (s_est > rhs) return fast_knapsack_eq<R>(row, hi, rhs, slots, counter, lane, thr);
    thr = make_thr(R(0), R(0), hi, 0, 0, hi, R(0));
    return kFastDone;
  } else {
    row.for_each([&](Data xd, int) {
      const R x = static_cast<R>(xd);
      if (x >= hi) ++n_hi;
      else if (x > R(0)) { ++n_mid; sum_mid += x; }
    });
    n_hi = warp_sum(n_hi); n_mid = warp_sum(n_mid); sum_mid = warp_sum(sum_mid);
  }
  const R s = sum_mid + hi * static_cast<R>(n_hi);
  if (s > rhs + eps) return fast_knapsack_eq<R>(row, hi, rhs, slots, counter, lane, thr);
  thr = make_thr(R(0), R(0), hi, n_hi, n_mid, hi, R(0));
  return kFastDone;
}

// The three knapsack operators with lo = 0 on a register row.  knapsack_le_biased
// (include/sdca/prox/knapsack_le_biased.h:89-129): rho = 0 is knapsack_le; otherwise the
// equality-constrained projection is the answer when its t >= rho * rhs, and the search over
// (U, M) -- the general routine -- is needed only below that.
template <typename R, int PROX, typename Data, int NV>
__device__ __forceinline__ FastStatus fast_knapsack_family(const RegRow<Data, NV>& row,
                                                           const ProxParams& q, Data* slots,
                                                           int* counter, int lane, Thr<R>& thr) {
  if (!(q.lo == 0 && q.hi > 0 && q.rhs > 0) || q.accurate) return kFastNeedsFullRow;
  const R hi = static_cast<R>(q.hi), rhs = static_cast<R>(q.rhs);
  if (PROX == kKnapsackEq) return fast_knapsack_eq<R>(row, hi, rhs, slots, counter, lane, thr);
  if (PROX == kKnapsackLe || q.rho == 0) return fast_knapsack_le<R>(row, hi, rhs, slots, counter, lane, thr);
  const R rho = static_cast<R>(q.rho);
  if (fast_knapsack_eq<R>(row, hi, rhs, slots, counter, lane, thr) != kFastDone) return kFastNeedsFullRow;
  const R eps = num<R>::eps() * max_(R(1), abs_(rhs));
  return (thr.t >= rho * rhs - eps) ? kFastDone : kFastNeedsFullRow;
}

// two_simplex (include/sdca/prox/two_simplex.h:18-119): the first phase projects each block
// onto the simplex of radius rhs on its own (:36-61) and is the answer when the two thresholds
// satisfy t + s >= -eps; that is the candidate path of fast_knapsack_eq run on each block with
// the other block's entries masked out.  Rows that need the joint second phase take the
// general routine.
template <typename R, typename Data, int NV>
__device__ __forceinline__ FastStatus fast_two_simplex(const RegRow<Data, NV>& row, int p, R rhs,
                                                       Data* slots, int* counter, int lane,
                                                       R& t_a, R& t_b) {
  if (!(rhs > 0)) return kFastNeedsFullRow;
  const R eps = num<R>::eps() * max_(R(1), rhs);
  constexpr int VN = RegRow<Data, NV>::VN;
  R t[2];
#pragma unroll
  for (int block = 0; block < 2; ++block) {
    RegRow<Data, NV> part;
    part.m = row.m;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      part.v[j] = row.v[j];
      Data* e = reinterpret_cast<Data*>(&part.v[j]);
#pragma unroll
      for (int c = 0; c < VN; ++c) {
        const bool first = ((j * 32 + lane) * VN + c) < p;
        if (first != (block == 0)) e[c] = -num<Data>::inf();
      }
    }
    Thr<R> thr;
    if (fast_knapsack_eq<R>(part, num<R>::inf(), rhs, slots, counter, lane, thr) != kFastDone)
      return kFastNeedsFullRow;
    t[block] = thr.t;
  }
  if (!(t[0] + t[1] >= -eps)) return kFastNeedsFullRow;
  t_a = t[0]; t_b = t[1];
  return kFastDone;
}

// ---- entropic projections of float rows --------------------------------------
// For float data the stated accuracy of outputs and thresholds is 1e-5, so the
// m exponentials of a log-sum-exp are evaluated in float (1e-7 each) and added
// up in R; everything after the sum (logarithms, the closed forms for t and hi)
// stays in R.  Double data keeps the general routines.

// max of the row and S = sum_i exp(a_i - max) (the maximum contributes exactly 1)
template <typename R, int NV>
__device__ __forceinline__ void row_max_and_expsum(const RegRow<float, NV>& row, float& mx,
                                                   float& lane_max, R& S) {
  float lm = -num<float>::inf();
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const float* e = reinterpret_cast<const float*>(&row.v[j]);
    lm = fmaxf(lm, fmaxf(fmaxf(e[0], e[1]), fmaxf(e[2], e[3])));
  }
  lane_max = lm;
  mx = warp_max_fast(lm);
  R acc0 = 0, acc1 = 0;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    // padding holds -inf: exp(-inf) = 0
    const float* e = reinterpret_cast<const float*>(&row.v[j]);
    const float p0 = exp_(e[0] - mx) + exp_(e[1] - mx);
    const float p1 = exp_(e[2] - mx) + exp_(e[3] - mx);
    acc0 += static_cast<R>(p0);
    acc1 += static_cast<R>(p1);
  }
  S = warp_sum(acc0 + acc1);
}

// Top-k entropy projection (include/sdca/prox/topk_entropy.h:20-76): the
// reference moves the current maximum into U and recomputes the log-sum-exp of
// the rest up to k - 1 times; here the k largest entries are sorted into lanes
// once and lane u evaluates "U = the u largest" from prefix sums of the
// exponentials, so all sizes of U are tested at the same time.
template <typename R, int NV>
__device__ __forceinline__ FastStatus fast_topk_entropy(const RegRow<float, NV>& row, int k,
                                                        float* slots, int* counter, int lane,
                                                        Thr<R>& thr) {
  const int m = row.size();
  if (k > 30 || m <= 32 || k > m) return kFastNeedsFullRow;
  const R eps = 16 * num<R>::eps();
  const R K = static_cast<R>(k);
  float mxf, lm;
  R S;
  row_max_and_expsum<R, NV>(row, mxf, lm, S);
  const R mx = static_cast<R>(mxf);
  R z = max_(S - R(1), R(0));
  R log_z = mx + log1p_(z);
  if (k <= 1 || mx - eps <= log_z - log_(K)) {
    const R e = exp_(-mx);
    const R log_z_1 = finite_(e) ? mx + log1p_(z + e) : R(0);
    thr = make_thr(log_z_1, R(0), R(1), 0, m, num<R>::inf(), -num<R>::inf());
    return kFastDone;
  }
  // the k + 1 largest entries, sorted, one per lane
  const float tau = kth_largest_of_lanes(lm, k, lane);
  const float cut = (tau > -num<float>::inf()) ? nextafterf(tau, -num<float>::inf()) : tau;
  LaneRow<float> cand;
  const int total = compact_candidates(row, cut, slots, counter, lane, cand);
  if (total > 32 || total <= k) return kFastNeedsFullRow;
  const Sorted<R> c = sort_candidates<R>(cand, total, lane);
  // prefix sums of exp(s_i - max) over the sorted candidates
  R pe = (lane < total) ? static_cast<R>(exp_(static_cast<float>(c.s) - mxf)) : R(0);
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const R up = __shfl_up_sync(kFullMask, pe, o);
    if (lane >= o) pe += up;
  }
  // lane u: U = the u largest; the rest has maximum s_u
  const int u = lane;
  const R pe_prev = __shfl_up_sync(kFullMask, pe, 1);        // sum of the first u exponentials
  const R s_prev = __shfl_up_sync(kFullMask, c.s, 1);        // smallest entry of U
  const R sumU_prev = __shfl_up_sync(kFullMask, c.P, 1);     // sum of U
  const bool active = (u >= 1) && (u <= k - 1) && (u < total);
  const R rest = S - pe_prev;                                // relative to the old maximum
  const R z_u = max_(rest * exp_(mx - c.s) - R(1), R(0));
  const R log_z_u = c.s + log1p_(z_u);
  const R tt = log_z_u - log_(K - static_cast<R>(u));
  const bool ok = active && (c.s - eps <= tt) && (tt <= s_prev + eps);
  // a rest that is a small fraction of the whole sum has lost too many digits
  const bool shaky = active && !(rest > R(1e-3) * S);
  if (__any_sync(kFullMask, shaky)) return kFastNeedsFullRow;
  const unsigned okmask = __ballot_sync(kFullMask, ok);
  const int last = min(k - 1, total - 1);
  const int ustar = okmask ? (__ffs(okmask) - 1) : last;     // the loop ends at k - 1 without a hit
  const R zs = __shfl_sync(kFullMask, z_u, ustar);
  const R log_zs = __shfl_sync(kFullMask, log_z_u, ustar);
  const R cur_max = __shfl_sync(kFullMask, c.s, ustar);
  const R min_U = __shfl_sync(kFullMask, s_prev, ustar);
  const R sum_U = __shfl_sync(kFullMask, sumU_prev, ustar);
  const R k_u = K - static_cast<R>(ustar);
  const R tmp = ((K - k_u) * log_zs + k_u * log_(k_u) - sum_U) / K;
  R t, hi;
  if (tmp > cur_max) {
    const R a = (1 + zs) * exp_(cur_max - tmp);
    t = tmp + log1p_(a * K) - log_(k_u);
    hi = a / (1 + a * K);
  } else {
    const R a = exp_(tmp - cur_max) / K;
    t = cur_max + log1p_(zs + a) - log_(k_u / K);
    hi = (1 + zs) / ((1 + zs + a) * K);
  }
  thr = make_thr(t, R(0), hi, ustar, m - ustar, min_U, -num<R>::inf());
  return kFastDone;
}

// Entropic projection (include/sdca/prox/entropy.h:19-53) when no entry reaches
// the upper bound, which one counting pass establishes; otherwise the general
// routine takes the row.
template <typename R, int NV>
__device__ __forceinline__ FastStatus fast_entropy(const RegRow<float, NV>& row, R hi, R rhs,
                                                   int lane, Thr<R>& thr) {
  const int m = row.size();
  const R eps = 16 * num<R>::eps() * max_(R(1), rhs);
  float mxf, lm;
  R S;
  row_max_and_expsum<R, NV>(row, mxf, lm, S);
  const R mx = static_cast<R>(mxf);
  const R t = (mx + log1p_(max_(S - R(1), R(0)))) - log_(rhs);
  const R tt = t + log_(hi) + eps;
  if (static_cast<R>(mxf) > tt) return kFastNeedsFullRow;
  thr = make_thr(t, R(0), hi, 0, m, num<R>::inf(), -num<R>::inf());
  return kFastDone;
}

// The general search for one row staged in shared memory; out of line so that
// the register budget of the kernel is set by the common path.
template <typename R, typename Data, int PROX>
__device__ __noinline__ Thr<R> full_row_thresholds(const Data* buf, int m, const ProxParams* q) {
  StridedRow<Data> view(buf, m);
  return compute_thresholds<R>(PROX, view, *q);
}

template <typename R, typename Data>
__device__ __noinline__ void full_row_two_simplex(const Data* buf, int m, int p, R rhs, R& t_a, R& t_b) {
  StridedRow<Data> ra(buf, p), rb(buf + p, m - p);
  const ThrPair<R> pr = thr_two_simplex<R>(ra, rb, rhs);
  t_a = pr.a.t; t_b = pr.b.t;
}

template <typename Data, typename R, int PROX, int NV>
__global__ void __launch_bounds__(kFastThreads, FastMinBlocks<Data, R, PROX, NV>::value)
fast_rows_kernel(const Data* a, Data* out, int m, long long n,
                 ProxParams q, int m_pad) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ Data slots_all[kFastThreads / 32][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps_per_block = kFastThreads / 32;
  __shared__ int counters[kFastThreads / 32];
  __shared__ R sorted_all[kFastThreads / 32][64];
  Data* slots = slots_all[warp];
  int* counter = &counters[warp];
  if (lane == 0) *counter = 0;
  __syncwarp();
  Data* stage = reinterpret_cast<Data*>(smem_raw) + static_cast<size_t>(warp) * m_pad;
  constexpr bool kTopk = (PROX == kTopkSimplex || PROX == kTopkSimplexBiased ||
                          PROX == kTopkCone || PROX == kTopkConeBiased);
  // operators with a fast path that can decline a row
  constexpr bool kKnap = (PROX == kKnapsackEq || PROX == kKnapsackLe || PROX == kKnapsackLeBiased);
  constexpr bool kStaged = kTopk || KnapsackStaged<PROX, NV>::value || PROX == kTwoSimplex ||
                           (std::is_same<Data, float>::value && (PROX == kTopkEntropy || PROX == kEntropy));
  const R rho_used = (PROX == kTopkSimplexBiased || PROX == kTopkConeBiased) ? static_cast<R>(q.rho) : R(0);
  const TopkConsts<R> tc(q.k > 0 ? q.k : 1, static_cast<R>(q.rhs), rho_used);
  for (long long r = static_cast<long long>(blockIdx.x) * warps_per_block + warp; r < n;
       r += static_cast<long long>(gridDim.x) * warps_per_block) {
    // top-k rows are read twice (the second time from L2): the search between the
    // two reads needs the registers more than it needs the row
    constexpr bool kTwice = kStaged;
    RegRow<Data, NV> row;
    row.m = m;
    if (kTwice) row.load_keep(a + r * m, lane); else row.load(a + r * m, lane);
    Thr<R> thr;
    FastStatus st = kFastNeedsFullRow;
    if (PROX == kTopkSimplex || PROX == kTopkSimplexBiased) {
      st = fast_topk_simplex<R>(row, q.k, static_cast<R>(q.rhs), rho_used, tc, slots, counter,
                                sorted_all[warp], lane, thr);
    } else if (PROX == kTopkCone || PROX == kTopkConeBiased) {
      st = (PROX == kTopkConeBiased && rho_used > 0)
               ? fast_topk_cone_biased<R>(row, q.k, rho_used, tc, slots, counter, sorted_all[warp], lane, thr)
               : fast_topk_cone<R>(row, q.k, rho_used, tc, slots, counter, sorted_all[warp], lane, thr);
    }
    if (kKnap && kStaged) st = fast_knapsack_family<R, PROX>(row, q, slots, counter, lane, thr);
    R t_a = 0, t_b = 0;   // two_simplex: the thresholds of the two blocks
    if (PROX == kTwoSimplex)
      st = fast_two_simplex<R>(row, static_cast<int>(q.p), static_cast<R>(q.rhs), slots, counter, lane, t_a, t_b);
    if (std::is_same<Data, float>::value && PROX == kTopkEntropy) {
      st = fast_topk_entropy<R, NV>(reinterpret_cast<const RegRow<float, NV>&>(row), q.k,
                                    reinterpret_cast<float*>(slots), counter, lane, thr);
    } else if (std::is_same<Data, float>::value && PROX == kEntropy) {
      st = fast_entropy<R, NV>(reinterpret_cast<const RegRow<float, NV>&>(row),
                               static_cast<R>(q.hi), static_cast<R>(q.rhs), lane, thr);
    }
    if (kStaged) {
      if (st != kFastDone) {
        if (kTwice) row.load(a + r * m, lane);
        row.for_each([&](Data x, int i) { stage[i] = x; });
        __syncwarp();
        if (PROX == kTwoSimplex)
          full_row_two_simplex<R, Data>(stage, m, static_cast<int>(q.p), static_cast<R>(q.rhs), t_a, t_b);
        else
          thr = full_row_thresholds<R, Data, PROX>(stage, m, &q);
        __syncwarp();
      }
    } else {
      bool done = false;
      if (kKnap) done = fast_knapsack_family<R, PROX>(row, q, slots, counter, lane, thr) == kFastDone;
      if (!done) thr = compute_thresholds<R>(PROX, row, q);
    }
    if (PROX == kTwoSimplex) {
      // x = clip(a - t, 0, rhs) on the first block, y = clip(b - s, 0, rhs) on the second
      const Data ta = static_cast<Data>(t_a), tb = static_cast<Data>(t_b), top = static_cast<Data>(static_cast<R>(q.rhs));
      const int p = static_cast<int>(q.p);
      RegRow<Data, NV> again;
      again.m = m;
      again.load(a + r * m, lane);
      again.store_indexed(out + r * m, lane,
                          [&](Data x, int i) { return clip_(x - (i < p ? ta : tb), Data(0), top); });
      continue;
    }
    Applier<Data> f(thr, prox_map(PROX), q.alpha);
    if (kTwice) {
      RegRow<Data, NV> again;
      again.m = m;
      again.load(a + r * m, lane);
      again.store(out + r * m, lane, f);
    } else {
      row.store(out + r * m, lane, f);
    }
  }
}

template <typename Data, typename R, int PROX, int NV>
int launch_fast(const Data* a, Data* out, int m, long long n, const ProxParams& q,
                cudaStream_t stream) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;
  auto kernel = fast_rows_kernel<Data, R, PROX, NV>;
  constexpr bool kTopk = (PROX == kTopkSimplex || PROX == kTopkSimplexBiased ||
                          PROX == kTopkCone || PROX == kTopkConeBiased) ||
                         (std::is_same<Data, float>::value && (PROX == kTopkEntropy || PROX == kEntropy));
  const int m_pad = (m + 15) & ~15;
  const size_t smem = (kTopk || KnapsackStaged<PROX, NV>::value || PROX == kTwoSimplex)
                          ? static_cast<size_t>(kFastThreads / 32) * m_pad * sizeof(Data) : 0;
  int per_sm = 0;
  SDCAB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kFastThreads, smem));
  if (per_sm < 1) per_sm = 1;
  const int warps = kFastThreads / 32;
  long long want = (n + warps - 1) / warps;
  int blocks = static_cast<int>(std::max<long long>(
      1, std::min<long long>(want, static_cast<long long>(per_sm) * info.sm_count)));
  kernel<<<blocks, kFastThreads, smem, stream>>>(a, out, m, n, q, m_pad);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

template <typename Data, typename R, int PROX>
int launch_fast_nv(const Data* a, Data* out, int m, long long n, const ProxParams& q,
                   cudaStream_t stream) {
  constexpr int VN = VecOf<Data>::N;
  const int vecs = (m + VN - 1) / VN;
  if (vecs <= 32 * 2) return launch_fast<Data, R, PROX, 2>(a, out, m, n, q, stream);
  if (vecs <= 32 * 4) return launch_fast<Data, R, PROX, 4>(a, out, m, n, q, stream);
  if (vecs <= 32 * 8) return launch_fast<Data, R, PROX, 8>(a, out, m, n, q, stream);
  return kNoFastPath;
}

// Register rows need 16-byte aligned rows: m a multiple of the vector width and
// aligned base pointers.
template <typename Data, typename R>
int launch_fast_rows(int prox, const Data* a, Data* out, int m, long long n,
                     const ProxParams& q, cudaStream_t stream) {
  constexpr int VN = VecOf<Data>::N;
  if (m % VN != 0 || m < 8) return kNoFastPath;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15) return kNoFastPath;
  switch (prox) {
    case kTopkSimplex: return launch_fast_nv<Data, R, kTopkSimplex>(a, out, m, n, q, stream);
    case kTopkCone: return launch_fast_nv<Data, R, kTopkCone>(a, out, m, n, q, stream);
    case kTopkSimplexBiased: return launch_fast_nv<Data, R, kTopkSimplexBiased>(a, out, m, n, q, stream);
    case kTopkConeBiased: return launch_fast_nv<Data, R, kTopkConeBiased>(a, out, m, n, q, stream);
    case kKnapsackEq: return launch_fast_nv<Data, R, kKnapsackEq>(a, out, m, n, q, stream);
    case kKnapsackLe: return launch_fast_nv<Data, R, kKnapsackLe>(a, out, m, n, q, stream);
    case kKnapsackLeBiased: return launch_fast_nv<Data, R, kKnapsackLeBiased>(a, out, m, n, q, stream);
    case kTwoSimplex: return launch_fast_nv<Data, R, kTwoSimplex>(a, out, m, n, q, stream);
    case kEntropy: return launch_fast_nv<Data, R, kEntropy>(a, out, m, n, q, stream);
    case kTopkEntropy: return launch_fast_nv<Data, R, kTopkEntropy>(a, out, m, n, q, stream);
    default: break;
  }
  return kNoFastPath;
}

}  // namespace sdcab
