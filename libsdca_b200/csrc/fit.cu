// SDCA fit on the device: solver::solve of the reference
// (include/sdca/solver.h:39-117) with update_variables
// (include/sdca/solver/update.h:52-107) as the step.
//
// The steps of an epoch form a sequential chain -- step s reads the variables
// step s-1 wrote -- but a step changes the dual variables of one example only,
// so the scores of the next 64 examples can be formed together, from the
// variables as they are now, by one product on the whole GPU (64 columns of K
// against A, or 64 examples against W); the chain itself then runs inside a
// single thread block that corrects the remaining score rows after every step
// by the one-example change (a 64 x 64 block of K, or of the examples' Gram
// matrix, is all it needs).  That turns N matrix-vector products per epoch into
// N / 64 matrix products and keeps the sequential part on chip.  For features
// the primal variables receive the block's rank-one changes afterwards, in
// step order.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <vector>

#include "common_host.h"
#include "eval_host.h"
#include "fit_host.h"
#include "gemm_blocked.cuh"
#include "primal.h"
#include "update_core.cuh"

namespace sdcab {
namespace {

constexpr int kFitThreads = 288;   // warp 0 steps, 256 threads keep the score rows current
constexpr int kBlockSteps = 64;   // steps whose score products are formed together

// ---- the chain ---------------------------------------------------------------
// One thread block walks through the `count` steps of a block of examples
// i_0, i_1, ...  It starts from S[b] = scores of example i_b under the variables
// the block began with; after step b changed a_{i_b} by delta, the scores of
// every later example of the block move by delta * G[b][b''], with
// G[b][b''] = K[i_b, i_b''] (kernel input) or -<x_{i_b}, x_{i_b''}> with
// delta = a_old - a_new (features, update.h:77-84), so S[b''] += delta * G[b][b'']
// keeps the rows current.  Rows are corrected in step order, which fixes the
// order of the floating-point sums.
struct ChainArgs {
  ObjectiveParams o;
  const int64_t* order;    // the block's examples: order[0 .. count)
  const int64_t* labels;
  const int64_t* offsets;  // multilabel objectives: the labels of example i are labels[offsets[i] .. offsets[i+1])
  double* S;               // count x m, scores at the start of the block (updated in place
                           // when they do not fit on chip)
  const double* G;         // kBlockSteps x kBlockSteps (row b = example i_b)
  void* A;                 // dual variables, n x m
  void* D;                 // features: count x m, a_old - a_new of every step (0 if skipped)
  double* t_keep;          // n: every example's threshold from its last step
  int m, count, kernel_input, s_on_chip;
};


constexpr int kSmallRow = 256;   // rows up to this length take the block-wide update

// Per-step constants of the update, worked out for all steps of a block at once.
template <typename R, typename Data>
struct StepConsts {
  Data norm2, alpha, beta;
  R rho, rho_inv;
};

// Warp sums of doubles through the integer reduction unit: every lane's term is
// scaled by a power of two to a 57-bit fixed-point number, the three 21-bit limbs
// are added by redux.sync, and the total is scaled back.  The sum is exact for
// the fixed-point terms, so it does not depend on the order of the lanes; the
// terms themselves are rounded at 2^-56 of `bound`, the same size as the
// rounding of a floating-point sum.  Takes a fifth of the shuffle butterfly's
// latency, which is what the step's chain of dependent reductions is made of.
struct FixedScale {
  double to_fixed, from_fixed;
};
// bound: a power of two not below any lane's |term|
__device__ __forceinline__ FixedScale fixed_scale(int bound_exponent) {
  FixedScale f;
  f.to_fixed = __hiloint2double((1023 + 56 - bound_exponent) << 20, 0);
  f.from_fixed = __hiloint2double((1023 - 56 + bound_exponent) << 20, 0);
  return f;
}
__device__ __forceinline__ double warp_sum_fixed(double v, const FixedScale& f) {
  const long long x = __double2ll_rn(v * f.to_fixed);
  const int l0 = static_cast<int>(x & 0x1fffff), l1 = static_cast<int>((x >> 21) & 0x1fffff),
            l2 = static_cast<int>(x >> 42);
  const long long s0 = __reduce_add_sync(0xffffffffu, l0), s1 = __reduce_add_sync(0xffffffffu, l1),
                  s2 = __reduce_add_sync(0xffffffffu, l2);
  return static_cast<double>(s0 + (s1 << 21) + (s2 << 42)) * f.from_fixed;
}
__device__ __forceinline__ float warp_sum_fixed(float v, const FixedScale& f) {
  return static_cast<float>(warp_sum_fixed(static_cast<double>(v), f));
}
// smallest e with |x| <= 2^e for every lane's x (finite)
__device__ __forceinline__ int warp_bound_exponent(double x) {
  const unsigned bits = __float_as_uint(__double2float_ru(fabs(x)));
  const unsigned top = __reduce_max_sync(0xffffffffu, bits);
  return static_cast<int>(top >> 23) - 127 + 1;
}

// f(t) = sum_i clip(v_i - t, 0, hi) over a row held in registers (NV entries per
// lane, -inf where the lane has none), with the sizes of the sets it is made of
// (u entries at hi, q entries above 0).
template <typename R>
struct ClipSum {
  R f;
  int u, q;
};
template <typename R, int NV>
__device__ __forceinline__ ClipSum<R> clip_sum(const R (&v)[NV], R t, R hi, const FixedScale& fs) {
  R x[NV];
  int cnt = 0;
#pragma unroll
  for (int e = 0; e < NV; ++e) {
    const R d = v[e] - t;
    x[e] = min_(max_(d, R(0)), hi);
    cnt += (d > R(0) ? 1 : 0) + (d >= hi ? 0x10000 : 0);
  }
  // pairwise, to keep the chain of dependent additions short
#pragma unroll
  for (int h = NV / 2; h > 0; h >>= 1) {
#pragma unroll
    for (int e = 0; e < h; ++e) x[e] += x[e + h];
  }
  ClipSum<R> out;
  out.f = warp_sum_fixed(x[0], fs);
  cnt = __reduce_add_sync(0xffffffffu, cnt);
  out.u = cnt >> 16; out.q = cnt & 0xffff;
  return out;
}

// The update of the top-k hinge (beta) objectives for one example by one warp with
// the row in registers: update_dual_variables of
// include/sdca/solver/objective/l2_topk_hinge.h:45-69,136-163, i.e.
// x = clip(v - t, 0, hi) solving  min 0.5 (|x|^2 + rho <1,x>^2) - <v,x>, <1,x> <= rhs
// (include/sdca/prox/knapsack_le_biased.h:96-127).  The reference first tries
// <1,x> = rhs by variable fixing, accepts it if t >= rho rhs, and otherwise
// searches sorted data for the sets at hi / strictly inside.  f is decreasing, so
// one evaluation at t = rho rhs tells the two cases apart: f >= rhs there means the
// equality case with its root to the right, anything else the root of
// t = rho f(t) to the left.  Either root is found by Newton steps on the
// piecewise-linear function -- a step is the closed form for the current sets, so
// the search ends as soon as a step stays on its piece -- kept inside a bracket,
// and t finally comes from the reference's closed form for the sets found.
// Lane l holds classes l, l + 32, ...; a_new receives their new variables.
// Returns false if the search did not settle (the caller then takes the general
// routine).
// What a step reads: the score row as the block's product left it, the change
// of the previous step that this row has not received yet (pending_g = 0 if
// none), the example's variables, and where the search for t starts.
template <typename R, typename Data>
struct StepInput {
  const double* Sb;        // scores of the example at the start of the block (+ earlier corrections)
  const double* pending;   // change of the previous step's variables (m entries)
  double pending_g;        // its factor for this row
  const Data* a_cur;       // current variables of the example
  int m, y;
  R t_start;
};

template <typename R, typename Data, int NV>
__device__ __forceinline__ bool warp_update_topk_hinge(const StepConsts<R, Data>& sc, R hi, R rhs,
                                                       const StepInput<R, Data>& in,
                                                       Data (&a_old)[NV], Data (&a_new)[NV],
                                                       R& t_out) {
  const int lane = threadIdx.x & 31;
  const int m = in.m, y = in.y;
  const R neg_inf = -num<R>::inf(), pos_inf = num<R>::inf();
  // the vector to project (objective/l2_topk_hinge.h:55-59)
  const Data score_y = static_cast<Data>(fma(in.pending[y], in.pending_g, in.Sb[y]));
  const Data vy = add_rn_(mul_rn_(sc.beta, in.a_cur[y]), mul_rn_(sc.alpha, score_y));
  const Data shift = sc.alpha - vy;
  Data vd[NV];
  R v[NV];
  double biggest = static_cast<double>(hi);
#pragma unroll
  for (int e = 0; e < NV; ++e) {
    const int j = lane + 32 * e;
    const bool mine = j < m && j != y;
    a_old[e] = j < m ? in.a_cur[j] : Data(0);
    const Data score = j < m ? static_cast<Data>(fma(in.pending[j], in.pending_g, in.Sb[j])) : Data(0);
    vd[e] = mine ? add_rn_(mul_rn_(sc.beta, a_old[e]), mul_rn_(sc.alpha, score)) + shift : Data(0);
    v[e] = mine ? static_cast<R>(vd[e]) : neg_inf;
    biggest = fmax(biggest, fabs(static_cast<double>(vd[e])));
  }
  // a lane's partial sums stay below NV * max(hi, |v|)
  const FixedScale fs = fixed_scale(warp_bound_exponent(biggest) + (NV == 8 ? 3 : 2));
  // Every solution has t >= 0.  The search starts from the threshold this example
  // had in the previous epoch (0 in the first), which late in a fit is nearly the
  // answer; t = rho rhs is only looked at when the steps get that far.
  const R rho = sc.rho, t_split = rho * rhs;
  R t = (in.t_start >= R(0) && in.t_start < t_split) ? in.t_start : R(0);
  R tl = neg_inf, tr = pos_inf;
  ClipSum<R> c = clip_sum<R, NV>(v, t, hi, fs);
  bool equality = false;
  // phi(t) = rhs - f(t) (equality) or t - rho f(t) (biased): increasing, root wanted
  bool settled = false;
  // The common course first, as a loop without side exits: t = rho f(t), Newton
  // steps that stay inside the bracket and left of rho rhs.  Anything else drops
  // into the general loop below with the state reached so far.
  for (int it = 0; it < 16; ++it) {
    const R phi = t - rho * c.f;
    const R slope = R(1) + rho * static_cast<R>(c.q - c.u);
    const R tn = t - phi / slope;
    const bool at_root = (phi == R(0)) || (tn == t);
    const R tl_n = phi < R(0) ? max_(tl, t) : tl, tr_n = phi < R(0) ? tr : min_(tr, t);
    const bool plain = tn > tl_n && tn < tr_n && tn < t_split;
    if (__any_sync(0xffffffffu, at_root || !plain)) break;
    tl = tl_n; tr = tr_n;
    const ClipSum<R> cn = clip_sum<R, NV>(v, tn, hi, fs);
    const bool same = (cn.u == c.u && cn.q == c.q);
    t = tn; c = cn;
    if (__any_sync(0xffffffffu, same)) { settled = true; break; }
  }
  for (int it = 0; it < 48 && !settled; ++it) {
    const int inside = c.q - c.u;
    const R phi = equality ? rhs - c.f : t - rho * c.f;
    if (phi == R(0)) { settled = true; break; }
    if (phi < R(0)) tl = max_(tl, t); else tr = min_(tr, t);
    R tn = t;
    bool newton = true;
    if (equality && inside == 0 && phi > R(0)) {
      newton = false;   // overshot into a flat stretch: halve the bracket instead
    } else if (equality && inside == 0) {
      // flat piece with f > rhs: the next piece starts where the first entries leave
      // the upper bound; solve on that piece
      R nb = pos_inf;
#pragma unroll
      for (int e = 0; e < NV; ++e) {
        const R b = v[e] - hi;
        if (b >= t) nb = min_(nb, b);
      }
      nb = -warp_max(-nb);
      if (!(nb < pos_inf)) return false;
      int leaving = 0;
#pragma unroll
      for (int e = 0; e < NV; ++e) leaving += (v[e] - hi == nb) ? 1 : 0;
      leaving = __reduce_add_sync(0xffffffffu, leaving);
      tn = nb + (c.f - rhs) / static_cast<R>(leaving);
    } else {
      const R slope = equality ? static_cast<R>(inside) : R(1) + rho * static_cast<R>(inside);
      tn = t - phi / slope;
      if (tn == t) { settled = true; break; }   // the root of this piece, to the last bit
    }
    bool probe = false;
    if (!equality && newton && tn >= t_split && t < t_split) {
      tn = t_split;      // which case it is shows at t = rho rhs
      probe = true;
      newton = false;
    } else if (!newton || !(tn > tl && tn < tr)) {
      if (!(tl > neg_inf) || !(tr < pos_inf)) return false;
      tn = tl + (tr - tl) / 2;
      newton = false;
      if (!(tn > tl && tn < tr)) return false;
    }
    const ClipSum<R> cn = clip_sum<R, NV>(v, tn, hi, fs);
    // a Newton step that finds the sets it started from has solved its piece exactly
    settled = newton && (cn.u == c.u && cn.q == c.q) && (!equality || inside > 0);
    t = tn; c = cn;
    if (probe && c.f >= rhs) {
      // the sum reaches rhs: the equality case, its root to the right of here
      equality = true;
      tl = t; tr = pos_inf;
    }
  }
  if (!settled) return false;
  // the reference's closed forms for the sets found (knapsack_le_biased.h:52;
  // knapsack_eq.h for the equality case): entries at hi, entries strictly inside
  const int inside = c.q - c.u;
  // the entries strictly inside add up to f + inside t - hi u  (f is their clipped sum)
  const R sum_inside = c.f + static_cast<R>(inside) * t - hi * static_cast<R>(c.u);
  if (equality) {
    if (inside > 0) t = (hi * static_cast<R>(c.u) + sum_inside - rhs) / static_cast<R>(inside);
  } else {
    t = (hi * static_cast<R>(c.u) + sum_inside) / (sc.rho_inv + static_cast<R>(inside));
  }
  // new variables (objective/l2_topk_hinge.h:64-68)
  const Data td = static_cast<Data>(t), hid = static_cast<Data>(hi);
  R part[NV];
#pragma unroll
  for (int e = 0; e < NV; ++e) {
    const int j = lane + 32 * e;
    const Data pj = (j < m && j != y) ? clip_(static_cast<Data>(vd[e] - td), Data(0), hid) : Data(0);
    part[e] = static_cast<R>(pj);
    a_new[e] = -pj;
  }
#pragma unroll
  for (int h = NV / 2; h > 0; h >>= 1) {
#pragma unroll
    for (int e = 0; e < h; ++e) part[e] += part[e + h];
  }
  const R total = warp_sum_fixed(part[0], fs);
  if ((y & 31) == lane) {
    const Data ay = static_cast<Data>(min_(rhs, total));
#pragma unroll
    for (int e = 0; e < NV; ++e) if (e == (y >> 5)) a_new[e] = ay;
  }
  t_out = t;
  return true;
}

// The general routine, out of line so that the chain's registers are set by the
// common path.
template <typename R, typename Data>
__device__ __noinline__ void general_update(const ObjectiveParams* o, Data norm2, const Data* scores,
                                            Data* a, Data* v, int m, int y) {
  update_dual_variables_multiclass<R, Data>(*o, norm2, scores, a, v, m, y);
}

// Where a step writes: the example's row of A, its change for the rows of S that
// follow, (features) the change for the primal variables, the threshold for the
// next epoch, and whether anything changed at all.
template <typename Data>
struct StepOutput {
  Data* a_row;
  double* delta;
  Data* d_row;       // features only
  double* t_keep;
  int* skip;
  int kernel_input;
};

template <typename R, typename Data>
__device__ __noinline__ void general_update_multilabel(const ObjectiveParams* o, Data norm2,
                                                       const Data* scores, Data* a, Data* v, int m,
                                                       const unsigned* mask, int num_labels) {
  update_dual_variables_multilabel_hinge<R, Data>(*o, norm2, scores, a, v, m, mask, num_labels);
}

// One step by warp 0 with the row in registers.
template <typename R, typename Data, int NV>
__device__ __forceinline__ bool warp_step_topk_hinge(const StepConsts<R, Data>& sc, R hi, R rhs,
                                                     const StepInput<R, Data>& in,
                                                     const StepOutput<Data>& out) {
  const int lane = threadIdx.x & 31;
  Data a_old[NV], a_new[NV];
  R t;
  if (!warp_update_topk_hinge<R, Data, NV>(sc, hi, rhs, in, a_old, a_new, t)) return false;
  if (lane == 0) *out.t_keep = static_cast<double>(t);
  if (out.kernel_input) {
#pragma unroll
    for (int e = 0; e < NV; ++e) {
      const int j = lane + 32 * e;
      if (j < in.m) {
        out.a_row[j] = a_new[e];
        out.delta[j] = static_cast<double>(a_new[e]) - static_cast<double>(a_old[e]);
      }
    }
    return true;
  }
  Data dlt[NV], asum = 0;
#pragma unroll
  for (int e = 0; e < NV; ++e) {
    dlt[e] = a_old[e] - a_new[e];   // var_copy of update.h:74-77 (0 past the row's end)
    asum += abs_(dlt[e]);
  }
  asum = warp_sum(asum);
  const bool moved = asum > num<Data>::eps();   // update.h:78
  if (!moved && lane == 0) *out.skip = 1;
#pragma unroll
  for (int e = 0; e < NV; ++e) {
    const int j = lane + 32 * e;
    if (j < in.m) {
      out.a_row[j] = a_new[e];
      out.delta[j] = static_cast<double>(dlt[e]);
      out.d_row[j] = moved ? dlt[e] : Data(0);
    }
  }
  return true;
}

// Rows of 129 .. 256 classes: the same step out of line, so that the registers of
// the chain are set by the short-row case.
template <typename R, typename Data>
__device__ __noinline__ bool warp_step_topk_hinge_long(const StepConsts<R, Data>* sc, R hi, R rhs,
                                                       const StepInput<R, Data>* in,
                                                       const StepOutput<Data>* out) {
  return warp_step_topk_hinge<R, Data, 8>(*sc, hi, rhs, *in, *out);
}

// ON_CHIP: the block's score rows live in shared memory (a compile-time fact, so
// that every access to them is a shared-memory instruction).
template <typename Data, typename R, bool ON_CHIP>
__global__ void __launch_bounds__(kFitThreads, 1) fit_chain_kernel(ChainArgs p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int m = p.m, count = p.count;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  double* G = reinterpret_cast<double*>(smem_raw);                  // 64 x 64
  double* delta = G + kBlockSteps * kBlockSteps;                    // 2 x m: this step's / the previous one's
  double* S = delta + 2 * m;                                        // count x m when on chip
  double* const S_shared = S;
  Data* scores = reinterpret_cast<Data*>(ON_CHIP ? S + static_cast<size_t>(kBlockSteps) * m : S);
  Data* a_s = scores + m;
  Data* v_s = a_s + m;
  Data* a_next = v_s + m;                                           // 2 x m, rows fetched ahead
  unsigned* label_mask = reinterpret_cast<unsigned*>(a_next + 2 * m);   // (m + 31) / 32 words (multilabel)
  const bool multilabel = objective_is_multilabel(p.o.id);
  __shared__ long long s_off[kBlockSteps];
  __shared__ long long s_idx[kBlockSteps];
  __shared__ int s_lab[kBlockSteps];
  __shared__ double s_t[kBlockSteps];
  __shared__ int s_skip[2];
  __shared__ StepConsts<R, Data> s_consts[kBlockSteps];
  const R hi_small = static_cast<R>(p.o.c) / static_cast<R>(p.o.k), rhs_small = static_cast<R>(p.o.c);
  const bool small_rows = (p.o.id == kObjL2TopkHinge || p.o.id == kObjL2TopkHingeSmooth) &&
                          m <= kSmallRow;
  Data* A = static_cast<Data*>(p.A);
  Data* D = static_cast<Data*>(p.D);

  for (int t = tid; t < kBlockSteps * kBlockSteps; t += kFitThreads) G[t] = p.G[t];
  for (int t = tid; t < 2 * m; t += kFitThreads) delta[t] = 0.0;
  if (tid < count) {
    const long long i = p.order[tid];
    s_idx[tid] = i;
    if (multilabel) {
      s_off[tid] = p.offsets[i];
      s_lab[tid] = static_cast<int>(p.offsets[i + 1] - p.offsets[i]);   // number of labels
    } else {
      s_lab[tid] = static_cast<int>(p.labels[i]);
    }
    s_t[tid] = p.t_keep[i];
  }
  if (tid < 2) s_skip[tid] = 1;
  if (ON_CHIP) {
    for (int t = tid; t < count * m; t += kFitThreads) S_shared[t] = p.S[t];
  } else {
    S = p.S;
  }
  __syncthreads();
  for (int j = tid; j < m; j += kFitThreads) a_next[j] = A[s_idx[0] * m + j];
  if (tid < count) {
    // constants of step tid (objective/l2_topk_hinge.h:53-54, 144-150; l2_hinge_topk.h alike)
    StepConsts<R, Data> sc;
    sc.norm2 = static_cast<Data>(p.kernel_input ? G[tid * kBlockSteps + tid] : -G[tid * kBlockSteps + tid]);
    const bool smooth = (p.o.id == kObjL2HingeTopkSmooth || p.o.id == kObjL2TopkHingeSmooth);
    const R c = static_cast<R>(p.o.c);
    sc.rho = smooth ? static_cast<R>(sc.norm2) / (static_cast<R>(sc.norm2) + static_cast<R>(p.o.gamma) / c) : R(1);
    sc.rho_inv = R(1) / sc.rho;
    sc.alpha = smooth ? static_cast<Data>(sc.rho) / sc.norm2 : Data(1) / sc.norm2;
    sc.beta = smooth ? -static_cast<Data>(sc.rho) : Data(-1);
    s_consts[tid] = sc;
  }
  __syncthreads();

  // Step b is worked by warp 0.  Meanwhile the other warps bring the rows after b
  // up to date with the change of step b - 1; row b itself receives that change
  // from warp 0 as it reads the row, so nobody waits for anybody inside a step.
  for (int b = 0; b < count; ++b) {
    const int cur = b & 1, prev = cur ^ 1;
    const bool pending = (b > 0) && (s_skip[prev] == 0);
    const double* d_prev = delta + prev * m;
    if (warp == 0) {
      const long long i = s_idx[b];
      const Data norm2 = s_consts[b].norm2;
      const bool active = norm2 > Data(0);    // update.h:63,97
      const Data* a_cur = a_next + cur * m;
      double* d_cur = delta + cur * m;
      Data* d_row = p.kernel_input ? nullptr : D + static_cast<size_t>(b) * m;
      if (lane == 0) s_skip[cur] = active ? 0 : 1;
      __syncwarp();
      bool done = !active;
      if (!active && d_row) {
        for (int j = lane; j < m; j += 32) d_row[j] = Data(0);
      }
      if (active && small_rows) {
        StepInput<R, Data> in;
        in.Sb = S + static_cast<size_t>(b) * m; in.pending = d_prev;
        in.pending_g = pending ? G[(b - 1) * kBlockSteps + b] : 0.0;
        in.a_cur = a_cur; in.m = m; in.y = s_lab[b]; in.t_start = static_cast<R>(s_t[b]);
        StepOutput<Data> out;
        out.a_row = A + i * m; out.delta = d_cur; out.d_row = d_row; out.t_keep = p.t_keep + i;
        out.skip = &s_skip[cur]; out.kernel_input = p.kernel_input;
        done = (m <= 128) ? warp_step_topk_hinge<R, Data, 4>(s_consts[b], hi_small, rhs_small, in, out)
                          : warp_step_topk_hinge_long<R, Data>(&s_consts[b], hi_small, rhs_small, &in, &out);
      }
      if (!done) {
        // the general routine on the row in shared memory
        const double* Sb = S + static_cast<size_t>(b) * m;
        const double g = pending ? G[(b - 1) * kBlockSteps + b] : 0.0;
        for (int j = lane; j < m; j += 32) {
          scores[j] = static_cast<Data>(fma(d_prev[j], g, Sb[j]));
          a_s[j] = a_cur[j];
        }
        __syncwarp();
        if (multilabel) {
          for (int w = lane; w < (m + 31) / 32; w += 32) label_mask[w] = 0u;
          __syncwarp();
          for (int g = lane; g < s_lab[b]; g += 32) {
            const int lab = static_cast<int>(p.labels[s_off[b] + g]);
            atomicOr(&label_mask[lab >> 5], 1u << (lab & 31));
          }
          __syncwarp();
          general_update_multilabel<R, Data>(&p.o, norm2, scores, a_s, v_s, m, label_mask, s_lab[b]);
        } else {
          general_update<R, Data>(&p.o, norm2, scores, a_s, v_s, m, s_lab[b]);
        }
        Data asum = 0;
        for (int j = lane; j < m; j += 32) {
          const Data a_new = a_s[j], a_old = a_cur[j];
          A[i * m + j] = a_new;
          if (p.kernel_input) {
            d_cur[j] = static_cast<double>(a_new) - static_cast<double>(a_old);
          } else {
            const Data dlt = a_old - a_new;   // var_copy of update.h:74-77
            asum += abs_(dlt);
            d_cur[j] = static_cast<double>(dlt);
          }
        }
        if (!p.kernel_input) {
          asum = warp_sum(asum);
          const bool moved = asum > num<Data>::eps();   // update.h:78
          if (!moved && lane == 0) s_skip[cur] = 1;
          for (int j = lane; j < m; j += 32) d_row[j] = moved ? static_cast<Data>(d_cur[j]) : Data(0);
        }
      }
    } else {
      const int h = tid - 32;
      if (h < 32 && b + 1 < count) {
        Data* nxt = a_next + prev * m;     // the buffer of step b + 1
        const Data* src = A + s_idx[b + 1] * m;
        for (int j = h; j < m; j += 32) nxt[j] = src[j];
      }
      if (pending) {
        // rows b + 1 .. move by the change of step b - 1 times G[b - 1][row]
        const double* Gp = G + (b - 1) * kBlockSteps;
        constexpr int kRowGroups = (kFitThreads - 32) >> 7, kFlight = 8;
        for (int j = h & 127; j < m; j += 128) {
          const double dj = d_prev[j];
          for (int first = b + 1 + (h >> 7); first < count; first += kFlight * kRowGroups) {
            double sv[kFlight], gv[kFlight];
#pragma unroll
            for (int r = 0; r < kFlight; ++r) {
              const int bb = first + r * kRowGroups;
              if (bb < count) {
                gv[r] = Gp[bb];
                sv[r] = S[static_cast<size_t>(bb) * m + j];
              }
            }
#pragma unroll
            for (int r = 0; r < kFlight; ++r) {
              const int bb = first + r * kRowGroups;
              if (bb < count) S[static_cast<size_t>(bb) * m + j] = fma(dj, gv[r], sv[r]);
            }
          }
        }
      }
    }
    __syncthreads();
  }
}

// S[b][j] = sum over the slices of the split product, plus (when the product
// left the previous block's examples out) those examples' share from their final
// variables: sum_b' A[i'_b'][j] * Gx[b'][b].  With G given it is filled as well:
// from the kernel matrix (kernel input) or from the sliced Gram product, negated
// (features).
template <typename Data>
struct PackArgs {
  const Data* s_parts; int slices; long long slice_stride;
  const Data* g_parts; int g_slices; long long g_stride;
  const Data* K; long long n;
  const int64_t* order; int count, m;
  double* S; double* G;
  const Data* A; const int64_t* prev_order; int prev_count; const double* Gx;
};

template <typename Data>
__global__ void __launch_bounds__(256) fit_pack_kernel(PackArgs<Data> p) {
  // 64 outputs per block, the terms of each dealt to four threads (term z to
  // thread z mod 4); the four partial sums are added in a fixed order
  __shared__ double part[4][64];
  const int lane64 = threadIdx.x & 63, group = threadIdx.x >> 6;
  const long long t = static_cast<long long>(blockIdx.x) * 64 + lane64;
  const long long s_elems = static_cast<long long>(p.count) * p.m;
  const long long u = t - s_elems;
  double acc = 0.0;
  if (t < s_elems) {
    for (int z = group; z < p.slices; z += 4) acc += static_cast<double>(p.s_parts[z * p.slice_stride + t]);
    if (p.prev_count > 0) {
      const int b = static_cast<int>(t / p.m), j = static_cast<int>(t % p.m);
      for (int bp = group; bp < p.prev_count; bp += 4)
        acc = fma(static_cast<double>(p.A[p.prev_order[bp] * p.m + j]), p.Gx[bp * kBlockSteps + b], acc);
    }
  } else if (p.G && u < kBlockSteps * kBlockSteps) {
    const int b = static_cast<int>(u / kBlockSteps), bb = static_cast<int>(u % kBlockSteps);
    if (b < p.count && bb < p.count) {
      if (p.K) {
        if (group == 0) acc = static_cast<double>(p.K[p.order[b] + p.n * p.order[bb]]);
      } else {
        for (int z = group; z < p.g_slices; z += 4)
          acc -= static_cast<double>(p.g_parts[z * p.g_stride + b * p.count + bb]);
      }
    }
  }
  part[group][lane64] = acc;
  __syncthreads();
  if (group != 0) return;
  const double total = (part[0][lane64] + part[1][lane64]) + (part[2][lane64] + part[3][lane64]);
  if (t < s_elems) p.S[t] = total;
  else if (p.G && u < kBlockSteps * kBlockSteps) p.G[u] = total;
}

// owner[i] = the block of 64 steps in which example i is visited this epoch
__global__ void fit_owner_kernel(const int64_t* __restrict__ order, long long n, int* __restrict__ owner) {
  const long long s = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (s < n) owner[order[s]] = static_cast<int>(s / kBlockSteps);
}

// G[b][b'] = K[i_b, i_b'] within a block and Gx[b'][b] = K[i'_b', i_b] from the
// previous block's examples to this block's (kernel input).
template <typename Data>
__global__ void fit_gather_kernel(const Data* __restrict__ K, long long n,
                                  const int64_t* __restrict__ order, int count,
                                  const int64_t* __restrict__ prev_order, int prev_count,
                                  double* __restrict__ G, double* __restrict__ Gx) {
  const int u = blockIdx.x * blockDim.x + threadIdx.x;
  const int which = u / (kBlockSteps * kBlockSteps), e = u % (kBlockSteps * kBlockSteps);
  const int r = e / kBlockSteps, c = e % kBlockSteps;
  if (which == 0) {
    G[e] = (r < count && c < count) ? static_cast<double>(K[order[r] + n * order[c]]) : 0.0;
  } else if (which == 1 && prev_count > 0) {
    Gx[e] = (r < prev_count && c < count) ? static_cast<double>(K[prev_order[r] + n * order[c]]) : 0.0;
  }
}

// W_j <- W_j - x_{i_b} * D[b][j] for the steps of one block in step order, every
// product and difference rounded on its own like the reference's ger (update.h:83).
template <typename Data>
__global__ void __launch_bounds__(256)
fit_primal_update_kernel(Data* W, const Data* __restrict__ X, const Data* __restrict__ D,
                         const int64_t* __restrict__ order, int count, int m, long long d) {
  __shared__ Data s_d[kBlockSteps];
  __shared__ long long s_i[kBlockSteps];
  const int j = blockIdx.y;
  if (threadIdx.x < count) {
    s_d[threadIdx.x] = D[static_cast<size_t>(threadIdx.x) * m + j];
    s_i[threadIdx.x] = order[threadIdx.x];
  }
  __syncthreads();
  const long long r = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (r >= d) return;
  Data w = W[d * j + r];
  for (int b = 0; b < count; ++b) {
    const Data dj = s_d[b];
    if (dj != Data(0)) w = sub_rn_(w, mul_rn_(X[d * s_i[b] + r], dj));
  }
  W[d * j + r] = w;
}

template <typename Data> int eval_sums_call(const sdcab_objective*, const sdcab_problem*, double*, void*);
template <> int eval_sums_call<float>(const sdcab_objective* o, const sdcab_problem* p, double* s, void* st) {
  return sdcab_eval_sums_f32_dev(o, p, s, nullptr, 0, st);
}
template <> int eval_sums_call<double>(const sdcab_objective* o, const sdcab_problem* p, double* s, void* st) {
  return sdcab_eval_sums_f64_dev(o, p, s, nullptr, 0, st);
}

struct DeviceBuffers {
  void* p[24] = {nullptr};
  int count = 0;
  cudaStream_t stream = nullptr, ahead = nullptr;
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t ev_product[2] = {nullptr, nullptr}, ev_steps[2] = {nullptr, nullptr}, ev_start = nullptr;
  ~DeviceBuffers() {
    for (int i = 0; i < count; ++i) cudaFree(p[i]);
    for (int i = 0; i < 4; ++i) if (ev[i]) cudaEventDestroy(ev[i]);
    for (int i = 0; i < 2; ++i) {
      if (ev_product[i]) cudaEventDestroy(ev_product[i]);
      if (ev_steps[i]) cudaEventDestroy(ev_steps[i]);
    }
    if (ev_start) cudaEventDestroy(ev_start);
    if (ahead) cudaStreamDestroy(ahead);
    if (stream) cudaStreamDestroy(stream);
  }
  template <typename T>
  int alloc(T** out, size_t elems) {
    void* ptr = nullptr;
    SDCAB_CUDA_TRY(cudaMalloc(&ptr, std::max<size_t>(elems, 1) * sizeof(T)));
    p[count++] = ptr;
    *out = static_cast<T*>(ptr);
    return SDCAB_OK;
  }
};

// The launches of one block of steps.
template <typename Data, typename R>
struct BlockRunner {
  ObjectiveParams o;
  const sdcab_problem* t;
  int sm_count = 0;
  size_t chain_smem = 0;
  int s_on_chip = 0;
  int slices = 1, g_slices = 1;
  int64_t* order = nullptr;     // the epoch's order on the device
  Data* s_parts = nullptr;      // slices x 64 x m
  Data* g_parts = nullptr;      // features: g_slices x 64 x 64
  double* S = nullptr;          // 64 x m
  double* G = nullptr;          // 64 x 64
  Data* D = nullptr;            // features: 64 x m
  double* t_keep = nullptr;     // n
  // kernel input, two of each: block b + 1's product is formed while block b steps
  Data* s_parts2[2] = {nullptr, nullptr};
  double* G2[2] = {nullptr, nullptr};
  double* Gx2[2] = {nullptr, nullptr};
  int* owner = nullptr;         // n

  static int pick_slices(int tiles, long long k, int bk, int sm_count) {
    long long want = (2LL * sm_count + tiles - 1) / tiles;
    const long long most = std::max<long long>(1, k / (4LL * bk));
    return static_cast<int>(std::max<long long>(1, std::min(want, most)));
  }

  int prepare(const DeviceInfo& info, DeviceBuffers& buf) {
    typedef SmallGemmTile<Data> GT;
    const long long m = t->m;
    sm_count = info.sm_count;
    const int tiles = static_cast<int>((m + GT::BN - 1) / GT::BN);
    slices = pick_slices(tiles, t->d, GT::BK, sm_count);
    g_slices = pick_slices(1, t->d, GT::BK, sm_count);
    const size_t fixed = (kBlockSteps * kBlockSteps + 2 * m) * sizeof(double) + 5 * m * sizeof(Data) +
                         static_cast<size_t>((m + 31) / 32 + 2) * sizeof(unsigned);
    const size_t with_s = fixed + static_cast<size_t>(kBlockSteps) * m * sizeof(double);
    s_on_chip = (with_s + 2048 <= info.smem_optin) ? 1 : 0;
    chain_smem = s_on_chip ? with_s : fixed;
    if (chain_smem + 2048 > info.smem_optin) return SDCAB_ERR_TOO_LARGE;
    if (s_on_chip)
      SDCAB_CUDA_TRY(cudaFuncSetAttribute(fit_chain_kernel<Data, R, true>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(chain_smem)));
    else
      SDCAB_CUDA_TRY(cudaFuncSetAttribute(fit_chain_kernel<Data, R, false>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(chain_smem)));
    int rc = buf.alloc(&order, static_cast<size_t>(t->n)); if (rc) return rc;
    if (t->input_kind == SDCAB_INPUT_KERNEL) {
      for (int h = 0; h < 2; ++h) {
        rc = buf.alloc(&s_parts2[h], static_cast<size_t>(slices) * kBlockSteps * m); if (rc) return rc;
        rc = buf.alloc(&G2[h], static_cast<size_t>(kBlockSteps) * kBlockSteps); if (rc) return rc;
        rc = buf.alloc(&Gx2[h], static_cast<size_t>(kBlockSteps) * kBlockSteps); if (rc) return rc;
      }
      rc = buf.alloc(&owner, static_cast<size_t>(t->n)); if (rc) return rc;
      s_parts = s_parts2[0];
    } else {
      rc = buf.alloc(&s_parts, static_cast<size_t>(slices) * kBlockSteps * m); if (rc) return rc;
    }
    rc = buf.alloc(&S, static_cast<size_t>(kBlockSteps) * m); if (rc) return rc;
    rc = buf.alloc(&G, static_cast<size_t>(kBlockSteps) * kBlockSteps); if (rc) return rc;
    rc = buf.alloc(&t_keep, static_cast<size_t>(t->n)); if (rc) return rc;
    SDCAB_CUDA_TRY(cudaMemsetAsync(t_keep, 0, static_cast<size_t>(t->n) * sizeof(double), buf.stream));
    if (t->input_kind != SDCAB_INPUT_KERNEL) {
      rc = buf.alloc(&g_parts, static_cast<size_t>(g_slices) * kBlockSteps * kBlockSteps); if (rc) return rc;
      rc = buf.alloc(&D, static_cast<size_t>(kBlockSteps) * m); if (rc) return rc;
    }
    return SDCAB_OK;
  }

  // steps [first, first + count) of the epoch whose order is on the device
  int run(long long first, int count, cudaStream_t s) const {
    typedef SmallGemmTile<Data> GT;
    const int m = static_cast<int>(t->m);
    const bool kernel_input = (t->input_kind == SDCAB_INPUT_KERNEL);
    const Data* X = static_cast<const Data*>(t->x);
    Data* A = static_cast<Data*>(const_cast<void*>(t->a));
    Data* W = static_cast<Data*>(const_cast<void*>(t->w));
    const int64_t* ord = order + first;
    GemmExtras x;
    x.a_gather = ord;
    x.slices = slices;
    x.c_slice_stride = static_cast<long long>(count) * m;
    int rc;
    if (kernel_input) {
      // S = K[:, block]' A : rows = columns of K (contiguous), A is n x m
      rc = launch_gemm_tile<Data, GT>(X, A, s_parts, count, m, static_cast<int>(t->n), t->n, m, m,
                                      false, s, x);
    } else {
      // S = X[:, block]' W, both with the feature index contiguous
      rc = launch_gemm_tile<Data, GT>(X, W, s_parts, count, m, static_cast<int>(t->d), t->d, t->d, m,
                                      true, s, x);
      if (rc) return rc;
      GemmExtras g;
      g.a_gather = ord; g.b_gather = ord; g.slices = g_slices;
      g.c_slice_stride = static_cast<long long>(count) * count;
      rc = launch_gemm_tile<Data, GT>(X, X, g_parts, count, count, static_cast<int>(t->d), t->d, t->d,
                                      count, true, s, g);
    }
    if (rc) return rc;
    const long long pack_threads = static_cast<long long>(count) * m + kBlockSteps * kBlockSteps;
    PackArgs<Data> pk;
    pk.s_parts = s_parts; pk.slices = slices; pk.slice_stride = x.c_slice_stride;
    pk.g_parts = g_parts; pk.g_slices = g_slices; pk.g_stride = static_cast<long long>(count) * count;
    pk.K = kernel_input ? X : nullptr; pk.n = t->n; pk.order = ord; pk.count = count; pk.m = m;
    pk.S = S; pk.G = G; pk.A = nullptr; pk.prev_order = nullptr; pk.prev_count = 0; pk.Gx = nullptr;
    fit_pack_kernel<Data><<<static_cast<unsigned>((pack_threads + 63) / 64), 256, 0, s>>>(pk);
    SDCAB_CUDA_TRY(cudaGetLastError());
    ChainArgs c;
    c.o = o; c.order = ord; c.labels = t->labels; c.offsets = t->offsets; c.S = S; c.G = G; c.A = A; c.D = D;
    c.t_keep = t_keep;
    c.m = m; c.count = count; c.kernel_input = kernel_input ? 1 : 0; c.s_on_chip = s_on_chip;
    if (s_on_chip) fit_chain_kernel<Data, R, true><<<1, kFitThreads, chain_smem, s>>>(c);
    else fit_chain_kernel<Data, R, false><<<1, kFitThreads, chain_smem, s>>>(c);
    SDCAB_CUDA_TRY(cudaGetLastError());
    if (!kernel_input) {
      dim3 grid(static_cast<unsigned>((t->d + 255) / 256), static_cast<unsigned>(m));
      fit_primal_update_kernel<Data><<<grid, 256, 0, s>>>(W, X, D, ord, count, m, t->d);
      SDCAB_CUDA_TRY(cudaGetLastError());
    }
    return SDCAB_OK;
  }

  // One epoch of a kernel-input fit with the products one block ahead of the
  // steps.  While block b steps on `sc`, block b + 1's product runs on `sg`
  // with block b's examples left out of A (their rows are being rewritten); their
  // share is added afterwards from their final variables (fit_pack_kernel).  Every
  // other row of A is final by then: the product waits for block b - 1's steps.
  int run_epoch_ahead(long long n, cudaStream_t sc, cudaStream_t sg, cudaEvent_t (&ev_product)[2],
                      cudaEvent_t (&ev_steps)[2], cudaEvent_t ev_start) const {
    typedef SmallGemmTile<Data> GT;
    const int m = static_cast<int>(t->m);
    const Data* K = static_cast<const Data*>(t->x);
    Data* A = static_cast<Data*>(const_cast<void*>(t->a));
    const long long blocks = (n + kBlockSteps - 1) / kBlockSteps;
    auto count_of = [&](long long b) { return static_cast<int>(std::min<long long>(kBlockSteps, n - b * kBlockSteps)); };
    fit_owner_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, sc>>>(order, n, owner);
    SDCAB_CUDA_TRY(cudaGetLastError());
    SDCAB_CUDA_TRY(cudaEventRecord(ev_start, sc));
    SDCAB_CUDA_TRY(cudaStreamWaitEvent(sg, ev_start, 0));
    auto product = [&](long long b) -> int {
      const int h = static_cast<int>(b & 1), count = count_of(b);
      const int64_t* ord = order + b * kBlockSteps;
      GemmExtras x;
      x.a_gather = ord; x.slices = slices;
      x.c_slice_stride = static_cast<long long>(count) * m;
      x.k_owner = owner; x.skip_owner = static_cast<int>(b - 1);   // -1 for the first block: nothing left out
      int rc = launch_gemm_tile<Data, GT>(K, A, s_parts2[h], count, m, static_cast<int>(t->n), t->n, m, m,
                                          false, sg, x);
      if (rc) return rc;
      fit_gather_kernel<Data><<<2 * kBlockSteps * kBlockSteps / 256, 256, 0, sg>>>(
          K, t->n, ord, count, b > 0 ? ord - kBlockSteps : nullptr, b > 0 ? kBlockSteps : 0, G2[h], Gx2[h]);
      SDCAB_CUDA_TRY(cudaGetLastError());
      SDCAB_CUDA_TRY(cudaEventRecord(ev_product[h], sg));
      return SDCAB_OK;
    };
    int rc = product(0);
    if (rc) return rc;
    for (long long b = 0; b < blocks; ++b) {
      const int h = static_cast<int>(b & 1), count = count_of(b);
      const int64_t* ord = order + b * kBlockSteps;
      SDCAB_CUDA_TRY(cudaStreamWaitEvent(sc, ev_product[h], 0));
      PackArgs<Data> pk;
      pk.s_parts = s_parts2[h]; pk.slices = slices; pk.slice_stride = static_cast<long long>(count) * m;
      pk.g_parts = nullptr; pk.g_slices = 0; pk.g_stride = 0; pk.K = nullptr; pk.n = t->n;
      pk.order = ord; pk.count = count; pk.m = m; pk.S = S; pk.G = nullptr;
      pk.A = A; pk.prev_order = b > 0 ? ord - kBlockSteps : nullptr; pk.prev_count = b > 0 ? kBlockSteps : 0;
      pk.Gx = Gx2[h];
      const long long pack_threads = static_cast<long long>(count) * m;
      fit_pack_kernel<Data><<<static_cast<unsigned>((pack_threads + 63) / 64), 256, 0, sc>>>(pk);
      SDCAB_CUDA_TRY(cudaGetLastError());
      SDCAB_CUDA_TRY(cudaEventRecord(ev_steps[h], sc));   // block b - 1 has stepped, block b's scores are packed
      ChainArgs c;
      c.o = o; c.order = ord; c.labels = t->labels; c.offsets = t->offsets; c.S = S; c.G = G2[h]; c.A = A;
      c.D = nullptr;
      c.t_keep = t_keep; c.m = m; c.count = count; c.kernel_input = 1; c.s_on_chip = s_on_chip;
      if (s_on_chip) fit_chain_kernel<Data, R, true><<<1, kFitThreads, chain_smem, sc>>>(c);
      else fit_chain_kernel<Data, R, false><<<1, kFitThreads, chain_smem, sc>>>(c);
      SDCAB_CUDA_TRY(cudaGetLastError());
      // The next product may start once block b - 1 has stepped; it is released
      // together with block b's steps (after the pack), on a stream of lower priority,
      // so that the stepping thread block holds its SM before the product's thread
      // blocks spread over the others.
      if (b + 1 < blocks) {
        SDCAB_CUDA_TRY(cudaStreamWaitEvent(sg, ev_steps[h], 0));
        rc = product(b + 1);
        if (rc) return rc;
      }
    }
    return SDCAB_OK;
  }
};

bool is_permutation(const int64_t* p, long long n, std::vector<unsigned char>& seen) {
  seen.assign(static_cast<size_t>(n), 0);
  for (long long i = 0; i < n; ++i) {
    const int64_t v = p[i];
    if (v < 0 || v >= n || seen[static_cast<size_t>(v)]) return false;
    seen[static_cast<size_t>(v)] = 1;
  }
  return true;
}

template <typename Data, typename R>
int fit_dev(const sdcab_objective* obj, const sdcab_problem* train, const sdcab_fit_criteria* crit,
            const int64_t* permutations, sdcab_eval_record* evals, int64_t evals_cap,
            sdcab_fit_result* result, cudaStream_t user_stream,
            const sdcab_fit_history* hist = nullptr) {
  const long long n = train->n, m = train->m;
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;

  DeviceBuffers buf;
  int prio_low = 0, prio_high = 0;
  SDCAB_CUDA_TRY(cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high));
  SDCAB_CUDA_TRY(cudaStreamCreateWithPriority(&buf.stream, cudaStreamNonBlocking, prio_high));
  SDCAB_CUDA_TRY(cudaStreamCreateWithPriority(&buf.ahead, cudaStreamNonBlocking, prio_low));
  for (int e = 0; e < 4; ++e) SDCAB_CUDA_TRY(cudaEventCreate(&buf.ev[e]));
  for (int e = 0; e < 2; ++e) {
    SDCAB_CUDA_TRY(cudaEventCreateWithFlags(&buf.ev_product[e], cudaEventDisableTiming));
    SDCAB_CUDA_TRY(cudaEventCreateWithFlags(&buf.ev_steps[e], cudaEventDisableTiming));
  }
  SDCAB_CUDA_TRY(cudaEventCreateWithFlags(&buf.ev_start, cudaEventDisableTiming));
  cudaStream_t s = buf.stream;
  // everything queued on the caller's stream so far comes first
  SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[0], user_stream));
  SDCAB_CUDA_TRY(cudaStreamWaitEvent(s, buf.ev[0], 0));

  BlockRunner<Data, R> runner;
  runner.o = to_params(obj);
  runner.t = train;
  rc = runner.prepare(info, buf);
  if (rc) return rc;
  double* sums_dev = nullptr;
  rc = buf.alloc(&sums_dev, static_cast<size_t>(SDCAB_EVAL_SUMS(m)));
  if (rc) return rc;

  // the reference's stopwatches run while it solves and evaluates (solver.h:81-131):
  // processor time by std::clock, wall time by a steady clock
  const std::clock_t cpu_begin = std::clock();
  const auto wall_begin = std::chrono::steady_clock::now();
  auto cpu_now = [&]() { return static_cast<double>(std::clock() - cpu_begin) / CLOCKS_PER_SEC; };
  auto wall_now = [&]() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - wall_begin).count();
  };
  int64_t epoch_now = 0;

  sdcab_problem ep = *train;
  ep.is_train = 1; ep.a_row_offset = 0; ep.include_primal_regularizer = 1;
  std::vector<double> sums(static_cast<size_t>(SDCAB_EVAL_SUMS(m)));
  std::vector<sdcab_eval_record> history;
  double eval_ms = 0, solve_ms = 0;
  auto evaluate = [&]() -> int {
    SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[2], s));
    int erc = SDCAB_OK;
    if (crit->recompute_primal && train->input_kind == SDCAB_INPUT_FEATURES) {
      // eval_recompute_primal (eval/core.h:148-182): W rebuilt from A, so that the
      // rounding of the steps' rank-one updates does not accumulate in it
      erc = primal_from_dual_dev<Data>(static_cast<const Data*>(train->x), static_cast<const Data*>(train->a),
                                       static_cast<const Data*>(train->w0),
                                       static_cast<Data*>(const_cast<void*>(train->w)), train->d, m, n, s);
      if (erc) return erc;
    }
    erc = eval_sums_call<Data>(obj, &ep, sums_dev, s);
    if (erc) return erc;
    SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[3], s));
    SDCAB_CUDA_TRY(cudaMemcpyAsync(sums.data(), sums_dev, sums.size() * sizeof(double),
                                   cudaMemcpyDeviceToHost, s));
    SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
    float ms = 0;
    SDCAB_CUDA_TRY(cudaEventElapsedTime(&ms, buf.ev[2], buf.ev[3]));
    eval_ms += ms;
    sdcab_eval_record rec;
    const int64_t slot = static_cast<int64_t>(history.size());
    const bool keep = hist && slot < hist->cap;
    erc = eval_finish(obj, m, sums.data(), &rec,
                      (keep && hist->train_accuracy) ? hist->train_accuracy + slot * m : nullptr);
    if (erc) return erc;
    history.push_back(rec);
    if (evals && static_cast<int64_t>(history.size()) <= evals_cap) evals[history.size() - 1] = rec;
    if (keep) {
      if (hist->train) hist->train[slot] = rec;
      if (hist->epoch) hist->epoch[slot] = epoch_now;
      if (hist->wall_seconds) hist->wall_seconds[slot] = wall_now();
    }
    // every held-out set after the training set (solver.h:124-131): scores from the
    // variables of the training problem, primal loss and accuracy / rank loss only
    if (hist && hist->tests) {
      for (int64_t ti = 0; ti < hist->num_tests; ++ti) {
        sdcab_problem tp = hist->tests[ti];
        tp.input_kind = train->input_kind; tp.is_train = 0; tp.d = train->d; tp.m = train->m;
        tp.a = train->a; tp.w = train->w; tp.w0 = nullptr; tp.a_row_offset = 0;
        tp.include_primal_regularizer = 0;
        SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[2], s));
        erc = eval_sums_call<Data>(obj, &tp, sums_dev, s);
        if (erc) return erc;
        SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[3], s));
        SDCAB_CUDA_TRY(cudaMemcpyAsync(sums.data(), sums_dev, sums.size() * sizeof(double),
                                       cudaMemcpyDeviceToHost, s));
        SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
        SDCAB_CUDA_TRY(cudaEventElapsedTime(&ms, buf.ev[2], buf.ev[3]));
        eval_ms += ms;
        sdcab_eval_record trec;
        double* acc = (keep && hist->test_accuracy)
                          ? hist->test_accuracy + (slot * hist->num_tests + ti) * m : nullptr;
        erc = eval_finish(obj, m, sums.data(), &trec, acc);
        if (erc) return erc;
        if (keep && hist->test) hist->test[slot * hist->num_tests + ti] = trec;
      }
    }
    return SDCAB_OK;
  };
  const double eps_floor = std::max(
      static_cast<double>(num<Data>::eps()), static_cast<double>(num<R>::eps()));
  auto check = [&](int status, int64_t epoch) {
    const sdcab_eval_record* last = history.empty() ? nullptr : &history.back();
    const sdcab_eval_record* before = history.size() > 1 ? &history[history.size() - 2] : nullptr;
    return check_stopping(status, last, before, crit->epsilon, epoch, crit->max_epoch, eps_floor,
                          crit->max_cpu_time, cpu_now(), crit->max_wall_time, wall_now());
  };

  // begin_solve (solver.h:59-80)
  int64_t epoch = 0;
  int status = (crit->max_epoch > 0) ? SDCAB_FIT_SOLVING : SDCAB_FIT_MAX_EPOCH;
  bool evaluated = false;
  if (crit->eval_on_start) {
    rc = evaluate(); if (rc) return rc;
    status = check(status, epoch);
  }

  MinstdRand gen;
  std::vector<int64_t> order_host(static_cast<size_t>(n));
  std::vector<unsigned char> seen;
  for (long long i = 0; i < n; ++i) order_host[static_cast<size_t>(i)] = i;

  while (status == SDCAB_FIT_SOLVING) {
    // begin_epoch (solver.h:94-100)
    evaluated = false;
    const int64_t* order_src;
    if (permutations) {
      order_src = permutations + epoch * n;
      if (!is_permutation(order_src, n, seen)) return SDCAB_ERR_ARG_RANGE;
    } else {
      shuffle_like_libstdcxx(order_host, gen);
      order_src = order_host.data();
    }
    SDCAB_CUDA_TRY(cudaMemcpyAsync(runner.order, order_src, static_cast<size_t>(n) * sizeof(int64_t),
                                   cudaMemcpyHostToDevice, s));
    SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[0], s));
    if (train->input_kind == SDCAB_INPUT_KERNEL) {
      rc = runner.run_epoch_ahead(n, s, buf.ahead, buf.ev_product, buf.ev_steps, buf.ev_start);
      if (rc) return rc;
    } else {
      for (long long first = 0; first < n; first += kBlockSteps) {
        rc = runner.run(first, static_cast<int>(std::min<long long>(kBlockSteps, n - first)), s);
        if (rc) return rc;
      }
    }
    SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[1], s));
    SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
    float ms = 0;
    SDCAB_CUDA_TRY(cudaEventElapsedTime(&ms, buf.ev[0], buf.ev[1]));
    solve_ms += ms;

    // end_epoch (solver.h:103-117)
    ++epoch;
    epoch_now = epoch;
    if (crit->eval_epoch > 0 && epoch % crit->eval_epoch == 0) {
      rc = evaluate(); if (rc) return rc;
      evaluated = true;
    }
    status = check(status, epoch);
  }
  // end_solve (solver.h:83-91)
  if (!evaluated && !(crit->eval_on_start && epoch == 0)) {
    rc = evaluate(); if (rc) return rc;
  }
  SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[1], s));
  SDCAB_CUDA_TRY(cudaStreamWaitEvent(user_stream, buf.ev[1], 0));
  SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
  if (result) {
    result->status = status; result->reserved = 0;
    result->epoch = epoch;
    result->num_evals = static_cast<int64_t>(history.size());
    result->solve_seconds = solve_ms * 1e-3;
    result->eval_seconds = eval_ms * 1e-3;
    result->cpu_seconds = cpu_now();
    result->wall_seconds = wall_now();
  }
  return SDCAB_OK;
}

int check_fit_args(const sdcab_objective* obj, const sdcab_problem* t, const sdcab_fit_criteria* c) {
  if (!obj || !t || !c) return SDCAB_ERR_ARG;
  if (t->n <= 0 || t->m <= 0 || t->d <= 0) return SDCAB_ERR_NOT_EMPTY;
  if (t->m < 2) return SDCAB_ERR_NUM_DIM;
  if (t->m > 0x7fffffffLL || t->d > 0x7fffffffLL) return SDCAB_ERR_TOO_LARGE;
  int rc = check_objective(obj, t->m);
  if (rc) return rc;
  if (!objective_has_update(obj->id)) return SDCAB_ERR_NOT_IMPLEMENTED;
  if (!t->x || !t->a || !t->labels) return SDCAB_ERR_ARG;
  if (objective_is_multilabel(obj->id) && !t->offsets) return SDCAB_ERR_ARG;
  if (t->input_kind == SDCAB_INPUT_KERNEL) {
    if (t->d != t->n) return SDCAB_ERR_NUM_DIM;
  } else if (t->input_kind == SDCAB_INPUT_FEATURES) {
    if (!t->w) return SDCAB_ERR_ARG;
  } else {
    return SDCAB_ERR_ARG;
  }
  if (!(c->epsilon >= 0) || c->max_epoch < 0 || c->eval_epoch < 0) return SDCAB_ERR_ARG_RANGE;
  if (!(c->max_cpu_time >= 0) || !(c->max_wall_time >= 0)) return SDCAB_ERR_ARG_RANGE;
  return SDCAB_OK;
}

int check_history(const sdcab_fit_history* h) {
  if (!h) return SDCAB_OK;
  if (h->cap < 0 || h->num_tests < 0) return SDCAB_ERR_ARG_RANGE;
  if (h->num_tests > 0 && !h->tests) return SDCAB_ERR_ARG;
  for (int64_t t = 0; t < h->num_tests; ++t) {
    if (h->tests[t].n <= 0) return SDCAB_ERR_NOT_EMPTY;
    if (!h->tests[t].x || !h->tests[t].labels) return SDCAB_ERR_ARG;
  }
  return SDCAB_OK;
}

template <typename Data>
int fit_entry(const sdcab_objective* obj, const sdcab_problem* t, const sdcab_fit_criteria* c,
              const int64_t* perm, sdcab_eval_record* evals, int64_t cap, sdcab_fit_result* res,
              void* stream, const sdcab_fit_history* hist = nullptr) {
  int rc = check_fit_args(obj, t, c);
  if (rc) return rc;
  rc = check_history(hist);
  if (rc) return rc;
  if (hist && objective_is_multilabel(obj->id))
    for (int64_t q = 0; q < hist->num_tests; ++q)
      if (!hist->tests[q].offsets) return SDCAB_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (obj->precision == SDCAB_PRECISION_FLOAT)
    return fit_dev<Data, float>(obj, t, c, perm, evals, cap, res, s, hist);
  return fit_dev<Data, double>(obj, t, c, perm, evals, cap, res, s, hist);
}

// Host buffers: copy the problem to the device, fit, copy the variables back.
template <typename Data>
int fit_host(const sdcab_objective* obj, const sdcab_problem* hp, const sdcab_fit_criteria* c,
             const int64_t* perm, sdcab_eval_record* evals, int64_t cap, sdcab_fit_result* res,
             const sdcab_fit_history* hist = nullptr) {
  int rc = check_fit_args(obj, hp, c);
  if (rc) return rc;
  rc = check_history(hist);
  if (rc) return rc;
  const long long n = hp->n, m = hp->m, d = hp->d;
  const bool kernel = (hp->input_kind == SDCAB_INPUT_KERNEL);
  const bool ml = objective_is_multilabel(obj->id);
  // the label checks of include/sdca/solver/data/output.h:169-215 (labels here are 0-based)
  rc = validate_labels(hp->labels, hp->offsets, n, m, ml);
  if (rc) return rc;
  const long long num_labels = ml ? hp->offsets[n] : n;
  DeviceBuffers buf;
  Data *dX = nullptr, *dA = nullptr, *dW = nullptr, *dW0 = nullptr;
  int64_t *dLab = nullptr, *dOff = nullptr;
  const size_t x_elems = static_cast<size_t>(n) * d, a_elems = static_cast<size_t>(n) * m,
               w_elems = static_cast<size_t>(d) * m;
  rc = buf.alloc(&dX, x_elems); if (rc) return rc;
  rc = buf.alloc(&dA, a_elems); if (rc) return rc;
  rc = buf.alloc(&dLab, static_cast<size_t>(num_labels)); if (rc) return rc;
  SDCAB_CUDA_TRY(cudaMemcpy(dX, hp->x, x_elems * sizeof(Data), cudaMemcpyHostToDevice));
  SDCAB_CUDA_TRY(cudaMemcpy(dA, hp->a, a_elems * sizeof(Data), cudaMemcpyHostToDevice));
  SDCAB_CUDA_TRY(cudaMemcpy(dLab, hp->labels, static_cast<size_t>(num_labels) * sizeof(int64_t),
                            cudaMemcpyHostToDevice));
  if (!kernel) {
    rc = buf.alloc(&dW, w_elems); if (rc) return rc;
    SDCAB_CUDA_TRY(cudaMemcpy(dW, hp->w, w_elems * sizeof(Data), cudaMemcpyHostToDevice));
    if (hp->w0) {
      // the proximal centre of a restarted fit (src/matlab/mex_solve.cpp:529-586): it enters
      // the primal regulariser of every evaluation and the rebuilt W
      rc = buf.alloc(&dW0, w_elems); if (rc) return rc;
      SDCAB_CUDA_TRY(cudaMemcpy(dW0, hp->w0, w_elems * sizeof(Data), cudaMemcpyHostToDevice));
    }
  }
  if (ml) {
    rc = buf.alloc(&dOff, static_cast<size_t>(n + 1)); if (rc) return rc;
    SDCAB_CUDA_TRY(cudaMemcpy(dOff, hp->offsets, static_cast<size_t>(n + 1) * sizeof(int64_t),
                              cudaMemcpyHostToDevice));
  }
  sdcab_problem dp = *hp;
  dp.x = dX; dp.a = dA; dp.w = dW; dp.w0 = dW0; dp.labels = dLab; dp.offsets = dOff;
  // held-out sets: checked like the training labels, then copied to the device
  std::vector<sdcab_problem> dtests;
  sdcab_fit_history dh;
  if (hist) {
    dh = *hist;
    for (int64_t q = 0; q < hist->num_tests; ++q) {
      const sdcab_problem& tp = hist->tests[q];
      if (ml && !tp.offsets) return SDCAB_ERR_ARG;
      rc = validate_labels(tp.labels, tp.offsets, tp.n, m, ml);
      if (rc) return rc;
      const long long tl = ml ? tp.offsets[tp.n] : tp.n;
      Data* tx = nullptr; int64_t *tlab = nullptr, *toff = nullptr;
      rc = buf.alloc(&tx, static_cast<size_t>(tp.n) * d); if (rc) return rc;
      rc = buf.alloc(&tlab, static_cast<size_t>(tl)); if (rc) return rc;
      SDCAB_CUDA_TRY(cudaMemcpy(tx, tp.x, static_cast<size_t>(tp.n) * d * sizeof(Data), cudaMemcpyHostToDevice));
      SDCAB_CUDA_TRY(cudaMemcpy(tlab, tp.labels, static_cast<size_t>(tl) * sizeof(int64_t), cudaMemcpyHostToDevice));
      if (ml) {
        rc = buf.alloc(&toff, static_cast<size_t>(tp.n + 1)); if (rc) return rc;
        SDCAB_CUDA_TRY(cudaMemcpy(toff, tp.offsets, static_cast<size_t>(tp.n + 1) * sizeof(int64_t), cudaMemcpyHostToDevice));
      }
      sdcab_problem q_dev = tp;
      q_dev.x = tx; q_dev.labels = tlab; q_dev.offsets = toff;
      dtests.push_back(q_dev);
    }
    dh.tests = dtests.empty() ? nullptr : dtests.data();
  }
  rc = fit_entry<Data>(obj, &dp, c, perm, evals, cap, res, nullptr, hist ? &dh : nullptr);
  if (rc) return rc;
  SDCAB_CUDA_TRY(cudaMemcpy(const_cast<void*>(hp->a), dA, a_elems * sizeof(Data), cudaMemcpyDeviceToHost));
  if (!kernel)
    SDCAB_CUDA_TRY(cudaMemcpy(const_cast<void*>(hp->w), dW, w_elems * sizeof(Data), cudaMemcpyDeviceToHost));
  return SDCAB_OK;
}

// matsdca_fit without Matlab: datasets + options in, model out.
template <typename Data>
int train_host(const sdcab_dataset* sets, int64_t num_sets, const sdcab_train_options* o, sdcab_model* model) {
  if (!sets || num_sets < 1 || !o || !model) return SDCAB_ERR_ARG;
  if (!model->A) return SDCAB_ERR_ARG;
  const sdcab_dataset& trn = sets[0];
  if (trn.n <= 0 || !trn.x || !trn.labels) return SDCAB_ERR_NOT_EMPTY;
  sdcab_objective obj;
  int rc = objective_from_name(o->objective ? o->objective : "msvm_smooth", o->c, o->gamma, o->k, &obj);
  if (rc) return rc;
  if (o->precision != SDCAB_PRECISION_DOUBLE && o->precision != SDCAB_PRECISION_FLOAT)
    return SDCAB_ERR_PRECISION;
  obj.precision = o->precision;
  const bool ml = objective_is_multilabel(obj.id);
  const bool kernel = o->is_dual != 0;
  const int64_t n = trn.n;
  const int64_t d = kernel ? n : o->num_dimensions;
  if (d <= 0) return SDCAB_ERR_NUM_DIM;
  if (!kernel && !model->W) return SDCAB_ERR_ARG;
  if (ml && !trn.offsets) return SDCAB_ERR_ARG;
  // labels: 0-based or 1-based, decided by the smallest training label
  // (validate_labels, include/sdca/solver/data/output.h:169-182); every set is shifted alike
  std::vector<std::vector<int64_t>> labels(static_cast<size_t>(num_sets));
  int64_t shift = 0, max_label = 0;
  for (int64_t q = 0; q < num_sets; ++q) {
    const sdcab_dataset& ds = sets[q];
    if (ds.n <= 0 || !ds.x || !ds.labels) return SDCAB_ERR_NOT_EMPTY;
    if (ml && !ds.offsets) return SDCAB_ERR_ARG;
    const int64_t count = ml ? ds.offsets[ds.n] : ds.n;
    if (count <= 0) return SDCAB_ERR_LABELS_RANGE;
    int64_t lo = ds.labels[0], hi = ds.labels[0];
    for (int64_t i = 1; i < count; ++i) { lo = std::min(lo, ds.labels[i]); hi = std::max(hi, ds.labels[i]); }
    if (q == 0) {
      if (lo != 0 && lo != 1) return SDCAB_ERR_LABELS_RANGE;
      shift = lo;
    }
    if (lo < shift) return SDCAB_ERR_LABELS_RANGE;
    max_label = std::max(max_label, hi - shift);
    labels[static_cast<size_t>(q)].assign(ds.labels, ds.labels + count);
    for (int64_t& v : labels[static_cast<size_t>(q)]) v -= shift;
  }
  const int64_t m = o->num_classes > 0 ? o->num_classes : max_label + 1;
  if (max_label >= m) return SDCAB_ERR_LABELS_RANGE;

  Data* A = static_cast<Data*>(model->A);
  Data* W = static_cast<Data*>(model->W);
  if (!o->warm_start) {
    std::fill(A, A + static_cast<size_t>(n) * m, Data(0));
    if (!kernel) {
      // W = W0 before the first step of a prox-regularised fit (mex_solve.cpp:566-571)
      if (o->W0) std::memcpy(W, o->W0, static_cast<size_t>(d) * m * sizeof(Data));
      else std::fill(W, W + static_cast<size_t>(d) * m, Data(0));
    }
  }
  sdcab_problem p = sdcab_problem();
  p.input_kind = kernel ? SDCAB_INPUT_KERNEL : SDCAB_INPUT_FEATURES;
  p.is_train = 1; p.d = d; p.n = n; p.m = m;
  p.x = trn.x; p.a = A; p.w = kernel ? nullptr : W; p.w0 = kernel ? nullptr : o->W0;
  p.labels = labels[0].data(); p.offsets = trn.offsets; p.include_primal_regularizer = 1;
  std::vector<sdcab_problem> tests;
  for (int64_t q = 1; q < num_sets; ++q) {
    sdcab_problem tp = sdcab_problem();
    tp.input_kind = p.input_kind; tp.d = d; tp.n = sets[q].n; tp.m = m;
    tp.x = sets[q].x; tp.labels = labels[static_cast<size_t>(q)].data(); tp.offsets = sets[q].offsets;
    tests.push_back(tp);
  }
  sdcab_fit_history h = model->history;
  h.num_tests = num_sets - 1;
  h.tests = tests.empty() ? nullptr : tests.data();
  sdcab_fit_result res = sdcab_fit_result();
  rc = fit_host<Data>(&obj, &p, &o->criteria, nullptr, nullptr, 0, &res, &h);
  if (rc) return rc;
  // the model (mex_solve.cpp:153-376)
  model->num_dimensions = d; model->num_examples = n; model->num_classes = m;
  model->is_dual = kernel ? 1 : 0; model->objective_id = obj.id;
  std::snprintf(model->objective, sizeof(model->objective), "%s", o->objective ? o->objective : "msvm_smooth");
  model->c = obj.c; model->gamma = obj.gamma; model->k = obj.k;
  model->criteria = o->criteria;
  model->status = res.status;
  model->data_precision = sizeof(Data) == 4 ? SDCAB_PRECISION_FLOAT : SDCAB_PRECISION_DOUBLE;
  model->precision = obj.precision;
  model->labels_one_based = static_cast<int32_t>(shift);
  model->epoch = res.epoch;
  model->cpu_time = res.cpu_seconds; model->wall_time = res.wall_seconds;
  model->solve_time = res.solve_seconds; model->eval_time = res.eval_seconds;
  model->num_evals = res.num_evals;
  model->history.num_tests = num_sets - 1;
  model->history.tests = nullptr;
  const int64_t last = std::min(res.num_evals, h.cap) - 1;
  model->relative_gap = (h.train && last >= 0) ? h.train[last].relative_gap : 0.0;
  return SDCAB_OK;
}

}  // namespace
}  // namespace sdcab


extern "C" {

int sdcab_epoch_permutations(int64_t n, int64_t num_epochs, int64_t* perm) {
  if (n < 0 || num_epochs < 0 || (!perm && n * num_epochs > 0)) return SDCAB_ERR_ARG;
  sdcab::epoch_permutations(n, num_epochs, perm);
  return SDCAB_OK;
}

int sdcab_fit_f32_dev(const sdcab_objective* obj, const sdcab_problem* train,
                      const sdcab_fit_criteria* criteria, const int64_t* permutations,
                      sdcab_eval_record* evals, int64_t evals_cap, sdcab_fit_result* result,
                      void* stream) {
  return sdcab::fit_entry<float>(obj, train, criteria, permutations, evals, evals_cap, result, stream);
}

int sdcab_fit_f64_dev(const sdcab_objective* obj, const sdcab_problem* train,
                      const sdcab_fit_criteria* criteria, const int64_t* permutations,
                      sdcab_eval_record* evals, int64_t evals_cap, sdcab_fit_result* result,
                      void* stream) {
  return sdcab::fit_entry<double>(obj, train, criteria, permutations, evals, evals_cap, result, stream);
}

int sdcab_fit_history_f32_dev(const sdcab_objective* obj, const sdcab_problem* train,
                              const sdcab_fit_criteria* criteria, const int64_t* permutations,
                              const sdcab_fit_history* history, sdcab_fit_result* result, void* stream) {
  return sdcab::fit_entry<float>(obj, train, criteria, permutations, nullptr, 0, result, stream, history);
}
int sdcab_fit_history_f64_dev(const sdcab_objective* obj, const sdcab_problem* train,
                              const sdcab_fit_criteria* criteria, const int64_t* permutations,
                              const sdcab_fit_history* history, sdcab_fit_result* result, void* stream) {
  return sdcab::fit_entry<double>(obj, train, criteria, permutations, nullptr, 0, result, stream, history);
}
int sdcab_fit_history_f32(const sdcab_objective* obj, const sdcab_problem* host_train,
                          const sdcab_fit_criteria* criteria, const int64_t* permutations,
                          const sdcab_fit_history* history, sdcab_fit_result* result) {
  return sdcab::fit_host<float>(obj, host_train, criteria, permutations, nullptr, 0, result, history);
}
int sdcab_fit_history_f64(const sdcab_objective* obj, const sdcab_problem* host_train,
                          const sdcab_fit_criteria* criteria, const int64_t* permutations,
                          const sdcab_fit_history* history, sdcab_fit_result* result) {
  return sdcab::fit_host<double>(obj, host_train, criteria, permutations, nullptr, 0, result, history);
}

void sdcab_train_options_default(sdcab_train_options* o) {
  if (!o) return;
  std::memset(o, 0, sizeof(*o));
  o->objective = nullptr; o->c = 1; o->gamma = 1; o->k = 1;
  o->is_dual = 0; o->precision = SDCAB_PRECISION_DOUBLE;
  // stopping_criteria of the reference (include/sdca/solver/solverdef.h:50-57)
  o->criteria.epsilon = 1e-3; o->criteria.max_epoch = 1000; o->criteria.eval_epoch = 10;
  o->criteria.eval_on_start = 0; o->criteria.recompute_primal = 0;
  o->criteria.max_cpu_time = 0; o->criteria.max_wall_time = 0;
}
int sdcab_train_f32(const sdcab_dataset* datasets, int64_t num_datasets,
                    const sdcab_train_options* options, sdcab_model* model) {
  return sdcab::train_host<float>(datasets, num_datasets, options, model);
}
int sdcab_train_f64(const sdcab_dataset* datasets, int64_t num_datasets,
                    const sdcab_train_options* options, sdcab_model* model) {
  return sdcab::train_host<double>(datasets, num_datasets, options, model);
}

int sdcab_fit_f32(const sdcab_objective* obj, const sdcab_problem* host_train,
                  const sdcab_fit_criteria* criteria, const int64_t* permutations,
                  sdcab_eval_record* evals, int64_t evals_cap, sdcab_fit_result* result) {
  return sdcab::fit_host<float>(obj, host_train, criteria, permutations, evals, evals_cap, result);
}

int sdcab_fit_f64(const sdcab_objective* obj, const sdcab_problem* host_train,
                  const sdcab_fit_criteria* criteria, const int64_t* permutations,
                  sdcab_eval_record* evals, int64_t evals_cap, sdcab_fit_result* result) {
  return sdcab::fit_host<double>(obj, host_train, criteria, permutations, evals, evals_cap, result);
}

}  // extern "C"
