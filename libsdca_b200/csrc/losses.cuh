// Per-example primal loss, conjugate (dual loss) and rank statistics of every
// objective, written for one lane group per example on top of thresholds.cuh.
//
// The reference swaps the ground-truth entries to the front of the score and
// dual vectors and then works on pointer ranges (include/sdca/solver/eval/
// primal.h:27-87, dual.h:23-63, data/output.h:42-165).  Here nothing is moved:
// views skip or select entries by index, which visits the same multisets.
#pragma once

#include "thresholds.cuh"

namespace sdcab {

enum ObjectiveId {
  kObjL2Entropy = 0,            // softmax
  kObjL2EntropyTopk,            // top-k softmax
  kObjL2HingeTopk,              // top-k hinge alpha
  kObjL2HingeTopkSmooth,
  kObjL2TopkHinge,              // top-k hinge beta; Crammer-Singer for k = 1
  kObjL2TopkHingeSmooth,
  kObjL2MultilabelHinge,
  kObjL2MultilabelHingeSmooth,
  kObjL2MultilabelEntropy,
  kNumObjectives
};

SDCAB_HD bool objective_is_multilabel(int id) { return id >= kObjL2MultilabelHinge; }

struct ObjectiveParams {
  int id;
  int k;
  double c, gamma;
};

// Factor applied to the summed primal loss (objective_base.h:108-128 with the
// constructors of each objective: l2_hinge_topk.h:29,114, l2_topk_hinge.h:30,117,
// l2_multilabel_hinge.h, l2_entropy*.h).
SDCAB_HD double objective_coeff(const ObjectiveParams& o) {
  switch (o.id) {
    case kObjL2HingeTopk: case kObjL2TopkHinge: return o.c / static_cast<double>(o.k);
    case kObjL2HingeTopkSmooth: case kObjL2TopkHingeSmooth: case kObjL2MultilabelHingeSmooth:
      return o.c / o.gamma;
    default: return o.c;
  }
}

// Entries selected by a bit mask (bit i of mask[i / 32]) and mapped by
// sign * x + shift in Data precision: the positive or the negative block of a
// multilabel example.
template <typename Data>
struct MaskedRow {
  typedef Data data_type;
  const Data* p;
  const unsigned* mask;
  int m, count;
  bool want;
  Data sign, shift;
  SDCAB_D int size() const { return count; }
  template <typename F>
  SDCAB_D void for_each(F&& f) const {
    for (int i = lane_id(); i < m; i += kLanes) {
      const bool bit = (mask[i >> 5] >> (i & 31)) & 1u;
      if (bit == want) f(static_cast<Data>(sign * p[i] + shift), i);
    }
  }
};

// <h, prox(h)> - 0.5 <prox(h), prox(h)> from the thresholds and the sets they
// describe (include/sdca/prox/proxdef.h:332-370), without forming prox(h).
template <typename R, typename Row>
SDCAB_D R smooth_loss_from_thresholds(const Row& row, const Thr<R>& t) {
  int cU = 0, cM = 0;
  R sU = 0, qU = 0, sM = 0, qM = 0, total = 0;
  row.for_each([&](typename Row::data_type xd, int) {
    const R x = static_cast<R>(xd);
    total += x;
    if (x > t.cutM) { ++cM; sM += x; qM += x * x; }
    if (x > t.cutU) { ++cU; sU += x; qU += x * x; }
  });
  cU = warp_sum(cU); cM = warp_sum(cM);
  sU = warp_sum(sU); qU = warp_sum(qU); sM = warp_sum(sM); qM = warp_sum(qM);
  total = warp_sum(total);
  const int n = row.size();
  R sum_U = 0, sq_U = 0;
  if (t.nU > 0) {
    const R fill = static_cast<R>(t.nU - cU);
    sum_U = sU + (fill != 0 ? fill * t.cutU : R(0));
    sq_U = qU + (fill != 0 ? fill * t.cutU * t.cutU : R(0));
  }
  R sum_UM = sum_U, sq_UM = sq_U;
  if (t.nM > 0) {
    const R fill = static_cast<R>(t.nU + t.nM - cM);
    sum_UM = sM + (fill != 0 ? fill * t.cutM : R(0));
    sq_UM = qM + (fill != 0 ? fill * t.cutM * t.cutM : R(0));
  }
  const R sum_M = sum_UM - sum_U, sq_M = sq_UM - sq_U, sum_L = total - sum_UM;
  const R num_hi = static_cast<R>(t.nU), num_mi = static_cast<R>(t.nM);
  const R num_lo = static_cast<R>(n - t.nU - t.nM);
  const R hp = t.hi * sum_U - t.t * sum_M + t.lo * sum_L + sq_M;
  const R pp = t.hi * t.hi * num_hi + t.t * t.t * num_mi + t.lo * t.lo * num_lo + sq_M -
               R(2) * t.t * sum_M;
  return hp - R(0.5) * pp;
}

// log(sum_i exp(s_i)) over a whole vector (math/log_exp.h:88-121)
template <typename R, typename Row>
SDCAB_D R row_log_sum_exp(const Row& row) {
  R mx, s; int cnt;
  row_max_sumexp<R>(row, [&](R, int) { return true; }, mx, s, cnt);
  return mx + log1p_(s);
}

// The k largest values of a row, summed (all of them, and only the positive ones).
// On the device every lane keeps the K largest of its own share in registers (a
// bubble through K slots per entry, in the data type), then the k largest of the
// whole row are popped off the lanes' heads; which of several equal values is
// taken does not matter to the sums.  K is the compile-time size that holds k.
#if defined(__CUDA_ARCH__)
__device__ __forceinline__ float lanes_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ double lanes_max(double v) { return warp_max(v); }

template <typename R, int K, typename Row>
__device__ __forceinline__ void topk_sums_device(const Row& row, int k, R& sum_all, R& sum_pos) {
  typedef typename Row::data_type Data;
  const Data none = -num<Data>::inf();
  Data top[K];
#pragma unroll
  for (int t = 0; t < K; ++t) top[t] = none;
  row.for_each([&](Data x, int) {
#pragma unroll
    for (int t = 0; t < K; ++t) {
      const Data hi = max_(top[t], x);
      x = min_(top[t], x);
      top[t] = hi;
    }
  });
  const int lane = lane_id();
  sum_all = 0; sum_pos = 0;
  for (int j = 0; j < k; ++j) {
    const Data best = lanes_max(top[0]);
    if (!(best > none)) break;                       // fewer than k entries
    const unsigned who = __ballot_sync(kFullMask, top[0] == best);
    if (lane == __ffs(who) - 1) {
#pragma unroll
      for (int t = 0; t + 1 < K; ++t) top[t] = top[t + 1];
      top[K - 1] = none;
    }
    const R v = static_cast<R>(best);
    sum_all += v;
    if (v > 0) sum_pos += v;
  }
}
#endif

// Sum of the k largest entries of the row and of the positive ones among them
// (the loop of include/sdca/solver/objective/l2_hinge_topk.h:71-86 on sorted data).
template <typename R, typename Row>
SDCAB_D void topk_sums(const Row& row, int k, R& sum_all, R& sum_pos) {
#if defined(__CUDA_ARCH__)
  if (k <= 8) {
    switch (k) {
      case 1: topk_sums_device<R, 1>(row, k, sum_all, sum_pos); return;
      case 2: topk_sums_device<R, 2>(row, k, sum_all, sum_pos); return;
      case 3: topk_sums_device<R, 3>(row, k, sum_all, sum_pos); return;
      case 4: topk_sums_device<R, 4>(row, k, sum_all, sum_pos); return;
      case 5: topk_sums_device<R, 5>(row, k, sum_all, sum_pos); return;
      case 6: topk_sums_device<R, 6>(row, k, sum_all, sum_pos); return;
      case 7: topk_sums_device<R, 7>(row, k, sum_all, sum_pos); return;
      default: topk_sums_device<R, 8>(row, k, sum_all, sum_pos); return;
    }
  }
#endif
  Taken<R> tk;
  sum_all = 0; sum_pos = 0;
  for (int j = 0; j < k; ++j) {
    R v;
    if (!take_next<R>(row, tk, v)) break;
    sum_all += v;
    if (v > 0) sum_pos += v;
  }
}

// ---- multiclass --------------------------------------------------------------
// s[0, m): scores of the example, y: its label.  Returns the primal loss before
// the objective's coefficient and the number of other classes scoring at least
// as high as the label (eval/primal.h:42-52).
template <typename R, typename Data>
SDCAB_D R multiclass_primal_loss(const ObjectiveParams& o, const Data* s, int m, int y, int& rank) {
  const Data sy = s[y];
  {
    int r = 0;
    for (int i = lane_id(); i < m; i += kLanes) r += (i != y && s[i] >= sy) ? 1 : 0;
    rank = warp_sum(r);
  }
  switch (o.id) {
    case kObjL2Entropy: {  // l2_entropy.h:77-91
      StridedRow<Data> all(s, m);
      return row_log_sum_exp<R>(all) - static_cast<R>(sy);
    }
    case kObjL2EntropyTopk: {  // l2_entropy_topk.h:74-94
      ShiftedRow<Data> h(s, m, y, static_cast<Data>(-sy));
      const Thr<R> t = thr_topk_entropy<R>(h, o.k);
      if (t.nU == 0) return t.t;
      int c; R sum_gt;
      row_count_sum_gt<R>(h, t.cutU, c, sum_gt);
      const R num_hi = static_cast<R>(t.nU);
      const R sum_hi = sum_gt + static_cast<R>(t.nU - c) * (t.nU > c ? t.cutU : R(0));
      const R K = static_cast<R>(o.k), sk = t.hi * K;
      return t.hi * (sum_hi + t.t * (K - num_hi)) - x_log_x(R(1) - sk) - num_hi * x_log_x(t.hi);
    }
    case kObjL2HingeTopk: case kObjL2TopkHinge: {  // l2_hinge_topk.h:71-86, l2_topk_hinge.h:72-87
      ShiftedRow<Data> h(s, m, y, static_cast<Data>(Data(1) - sy));
      R sum_all, sum_pos;
      topk_sums<R>(h, o.k, sum_all, sum_pos);
      return (o.id == kObjL2HingeTopk) ? max_(R(0), sum_all) : sum_pos;
    }
    case kObjL2HingeTopkSmooth: {  // l2_hinge_topk.h:162-179
      ShiftedRow<Data> h(s, m, y, static_cast<Data>(Data(1) - sy));
      const Thr<R> t = thr_topk_simplex<R>(h, o.k, static_cast<R>(o.gamma), R(0));
      return smooth_loss_from_thresholds<R>(h, t);
    }
    case kObjL2TopkHingeSmooth: {  // l2_topk_hinge.h:166-183
      ShiftedRow<Data> h(s, m, y, static_cast<Data>(Data(1) - sy));
      const R gamma = static_cast<R>(o.gamma);
      const Thr<R> t = thr_knapsack_le<R>(h, R(0), gamma / static_cast<R>(o.k), gamma);
      return smooth_loss_from_thresholds<R>(h, t);
    }
    default: break;
  }
  return R(0);
}

// a[0, m): dual variables of the example (a[y] >= 0, the others <= 0).
template <typename R, typename Data>
SDCAB_D R multiclass_dual_loss(const ObjectiveParams& o, const Data* a, int m, int y) {
  const R c = static_cast<R>(o.c);
  switch (o.id) {
    case kObjL2HingeTopk: case kObjL2TopkHinge:  // objective_base.h:49-56
      return static_cast<R>(a[y]);
    case kObjL2HingeTopkSmooth: case kObjL2TopkHingeSmooth: {  // l2_hinge_topk.h:182-192
      R dot = 0;
      for (int i = lane_id(); i < m; i += kLanes)
        if (i != y) dot += static_cast<R>(a[i]) * static_cast<R>(a[i]);
      dot = warp_sum(dot);
      return static_cast<R>(a[y]) - static_cast<R>(o.gamma) / (R(2) * c) * dot;
    }
    case kObjL2Entropy: case kObjL2EntropyTopk: {  // l2_entropy.h:94-114, l2_entropy_topk.h:97-107
      R acc = 0;
      for (int i = lane_id(); i < m; i += kLanes)
        if (i != y) acc += x_log_x(-static_cast<R>(a[i]));
      acc = warp_sum(acc);
      const R ay = static_cast<R>(a[y]);
      if (o.id == kObjL2EntropyTopk) return x_log_x(c) - x_log_x(c - ay) - acc;
      // general form with one label: log(p) = 0
      return -x_log_x(c - ay) - acc + x_log_x(c) + log_(R(1)) * (c - ay);
    }
    default: break;
  }
  return R(0);
}

// ---- multilabel --------------------------------------------------------------
// mask marks the nl positive classes; labels[0, nl) lists them.
template <typename R, typename Data>
SDCAB_D R multilabel_primal_loss(const ObjectiveParams& o, const Data* s, int m,
                                 const unsigned* mask, const long long* labels, int nl,
                                 R& rank_loss) {
  // eval/primal.h:67-80: sum over positives of #{negatives scoring >= it}
  {
    R rl = 0;
    for (int g = 0; g < nl; ++g) {
      const Data sg = s[labels[g]];
      int cnt = 0;
      for (int i = lane_id(); i < m; i += kLanes) {
        const bool pos = (mask[i >> 5] >> (i & 31)) & 1u;
        cnt += (!pos && s[i] >= sg) ? 1 : 0;
      }
      rl += static_cast<R>(warp_sum(cnt));
    }
    rank_loss = rl / static_cast<R>(static_cast<long long>(nl) * (m - nl));
  }
  switch (o.id) {
    case kObjL2MultilabelEntropy: {  // l2_multilabel_entropy.h:72-86
      StridedRow<Data> all(s, m);
      R sum_pos = 0;
      for (int g = lane_id(); g < nl; g += kLanes) sum_pos += static_cast<R>(s[labels[g]]);
      sum_pos = warp_sum(sum_pos);
      return row_log_sum_exp<R>(all) - sum_pos / static_cast<R>(nl);
    }
    case kObjL2MultilabelHinge: {  // l2_multilabel_hinge.h:69-84
      Data min_pos = num<Data>::inf(), max_neg = -num<Data>::inf();
      for (int i = lane_id(); i < m; i += kLanes) {
        const bool pos = (mask[i >> 5] >> (i & 31)) & 1u;
        if (pos) min_pos = min_(min_pos, s[i]); else max_neg = max_(max_neg, s[i]);
      }
      min_pos = warp_min(min_pos); max_neg = warp_max(max_neg);
      return max_(R(0), static_cast<R>(max_neg - min_pos + Data(1)));
    }
    case kObjL2MultilabelHingeSmooth: {  // l2_multilabel_hinge.h:168-191
      MaskedRow<Data> pos, neg;
      pos.p = s; pos.mask = mask; pos.m = m; pos.count = nl; pos.want = true;
      pos.sign = Data(-1); pos.shift = Data(0.5);
      neg.p = s; neg.mask = mask; neg.m = m; neg.count = m - nl; neg.want = false;
      neg.sign = Data(1); neg.shift = Data(0.5);
      const ThrPair<R> t = thr_two_simplex<R>(pos, neg, static_cast<R>(o.gamma));
      return smooth_loss_from_thresholds<R>(pos, t.a) + smooth_loss_from_thresholds<R>(neg, t.b);
    }
    default: break;
  }
  return R(0);
}

template <typename R, typename Data>
SDCAB_D R multilabel_dual_loss(const ObjectiveParams& o, const Data* a, int m,
                               const unsigned* mask, int nl) {
  const R c = static_cast<R>(o.c);
  R sum_pos = 0, sum_neg = 0, dot = 0, ent_pos = 0, ent_neg = 0;
  const R p = static_cast<R>(nl);
  for (int i = lane_id(); i < m; i += kLanes) {
    const bool pos = (mask[i >> 5] >> (i & 31)) & 1u;
    const R v = static_cast<R>(a[i]);
    dot += v * v;
    if (pos) { sum_pos += v; ent_pos += x_log_x(c - p * v); }
    else { sum_neg += v; ent_neg += x_log_x(-v); }
  }
  sum_pos = warp_sum(sum_pos); sum_neg = warp_sum(sum_neg); dot = warp_sum(dot);
  switch (o.id) {
    case kObjL2MultilabelHinge: return sum_pos;  // l2_multilabel_hinge.h:87-96
    case kObjL2MultilabelHingeSmooth:            // l2_multilabel_hinge.h:194-208
      return R(0.5) * (sum_pos - sum_neg - static_cast<R>(o.gamma) / c * dot);
    case kObjL2MultilabelEntropy: {              // l2_multilabel_entropy.h:89-109
      ent_pos = warp_sum(ent_pos); ent_neg = warp_sum(ent_neg);
      return -ent_pos / p - ent_neg + x_log_x(c) + log_(p) * (c - sum_pos);
    }
    default: break;
  }
  return R(0);
}

}  // namespace sdcab
