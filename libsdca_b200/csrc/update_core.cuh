// One SDCA step on the dual variables of one example, for the hinge family of
// objectives (top-k hinge alpha / beta, smooth or not; Crammer-Singer is beta
// with k = 1) and the top-k softmax, written for one lane group on top of
// thresholds.cuh.
//
// Follows update_dual_variables of the reference's objectives
// (include/sdca/solver/objective/l2_topk_hinge.h:45-69,136-163,
// l2_hinge_topk.h:43-68,131-159 and l2_entropy_topk.h:46-71): build the vector to
// project from the scores and the current variables in data precision, project it
// (knapsack_le_biased, topk_simplex_biased or topk_entropy_biased), read the new
// variables off the projection.  The reference moves the label to the front
// first; here the label index is skipped.
#pragma once

#include "losses.cuh"
#include "prox_core.cuh"

namespace sdcab {

// Products and sums that must round separately (the reference's BLAS-1 calls are
// separate loops); on the device the compiler would contract them otherwise.
SDCAB_HD float mul_rn_(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}
SDCAB_HD double mul_rn_(double a, double b) {
#if defined(__CUDA_ARCH__)
  return __dmul_rn(a, b);
#else
  return a * b;
#endif
}
SDCAB_HD float add_rn_(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fadd_rn(a, b);
#else
  return a + b;
#endif
}
SDCAB_HD double add_rn_(double a, double b) {
#if defined(__CUDA_ARCH__)
  return __dadd_rn(a, b);
#else
  return a + b;
#endif
}
template <typename T> SDCAB_HD T sub_rn_(T a, T b) { return add_rn_(a, -b); }

SDCAB_HD bool objective_has_update(int id) { return id >= 0 && id < kNumObjectives; }

// Softmax and multilabel softmax (include/sdca/solver/objective/l2_entropy.h:47-74,
// l2_multilabel_entropy.h:42-69): v = scores - norm2 * a, the labels' block and the
// others' block are projected together by prox_two_entropy with alpha = c * norm2;
// a_label = -c x + c / (number of labels), a_other = -c x.  RowP / RowN view the two
// blocks of v; `is_label(j)` tells them apart when the new variables are written.
template <typename R, typename Data, typename RowP, typename RowN, typename IsLabel>
SDCAB_D void finish_entropy_update(const ObjectiveParams& o, Data norm2, const RowP& pos,
                                   const RowN& neg, int num_labels, const Data* v, Data* a, int m,
                                   IsLabel is_label) {
  const R c = static_cast<R>(o.c);
  const R alpha = c * static_cast<R>(norm2);
  const ThrPair<R> thr = thr_two_entropy<R>(pos, neg, alpha);
  Applier<Data> fp(thr.a, kMapScaledLambert, static_cast<double>(alpha));
  Applier<Data> fn(thr.b, kMapScaledLambert, static_cast<double>(alpha));
  const Data minus_c = static_cast<Data>(-c);
  const Data share = static_cast<Data>(c / static_cast<R>(num_labels));
  for (int j = lane_id(); j < m; j += kLanes) {
    a[j] = is_label(j) ? add_rn_(mul_rn_(minus_c, fp(v[j])), share) : mul_rn_(minus_c, fn(v[j]));
  }
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
}

template <typename R, typename Data>
SDCAB_D void update_dual_variables_multilabel_entropy(const ObjectiveParams& o, Data norm2,
                                                      const Data* scores, Data* a, Data* v, int m,
                                                      const unsigned* mask, int num_labels) {
  for (int j = lane_id(); j < m; j += kLanes) v[j] = add_rn_(mul_rn_(-norm2, a[j]), scores[j]);
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  MaskedRow<Data> pos, neg;
  pos.p = v; pos.mask = mask; pos.m = m; pos.count = num_labels; pos.want = true;
  pos.sign = Data(1); pos.shift = Data(0);
  neg = pos; neg.count = m - num_labels; neg.want = false;
  finish_entropy_update<R, Data>(o, norm2, pos, neg, num_labels, v, a, m,
                                 [&](int j) { return ((mask[j >> 5] >> (j & 31)) & 1u) != 0; });
}

template <typename R, typename Data>
SDCAB_D void update_dual_variables_entropy(const ObjectiveParams& o, Data norm2, const Data* scores,
                                           Data* a, Data* v, int m, int y) {
  for (int j = lane_id(); j < m; j += kLanes) v[j] = add_rn_(mul_rn_(-norm2, a[j]), scores[j]);
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  OneEntryRow<Data> pos;
  pos.x = v[y]; pos.index = y;
  ShiftedRow<Data> neg(v, m, y, Data(0));
  finish_entropy_update<R, Data>(o, norm2, pos, neg, 1, v, a, m, [&](int j) { return j == y; });
}

// Multilabel hinge, smooth or not (include/sdca/solver/objective/l2_multilabel_hinge.h:39-66,
// 136-165): v = alpha * scores - beta * a; the labels' entries become alpha/2 - v, the others
// alpha/2 + v; both blocks are projected together by prox_two_simplex with radius c; the
// labels keep the projection, the others its negative.  `mask` has bit j set for the labels.
template <typename R, typename Data>
SDCAB_D void update_dual_variables_multilabel_entropy(const ObjectiveParams& o, Data norm2,
                                                      const Data* scores, Data* a, Data* v, int m,
                                                      const unsigned* mask, int num_labels);

template <typename R, typename Data>
SDCAB_D void update_dual_variables_multilabel_hinge(const ObjectiveParams& o, Data norm2,
                                                    const Data* scores, Data* a, Data* v, int m,
                                                    const unsigned* mask, int num_labels) {
  if (o.id == kObjL2MultilabelEntropy) {
    update_dual_variables_multilabel_entropy<R, Data>(o, norm2, scores, a, v, m, mask, num_labels);
    return;
  }
  const R c = static_cast<R>(o.c);
  const bool smooth = (o.id == kObjL2MultilabelHingeSmooth);
  const R denom = static_cast<R>(norm2) + static_cast<R>(o.gamma) / c;
  const Data alpha = smooth ? static_cast<Data>(R(1) / denom) : Data(1) / norm2;
  const Data beta = smooth ? static_cast<Data>(static_cast<R>(norm2) / denom) : Data(1);
  for (int j = lane_id(); j < m; j += kLanes) v[j] = add_rn_(mul_rn_(-beta, a[j]), mul_rn_(alpha, scores[j]));
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  const Data half = alpha / 2;
  MaskedRow<Data> pos, neg;
  pos.p = v; pos.mask = mask; pos.m = m; pos.count = num_labels; pos.want = true;
  pos.sign = Data(-1); pos.shift = half;
  neg.p = v; neg.mask = mask; neg.m = m; neg.count = m - num_labels; neg.want = false;
  neg.sign = Data(1); neg.shift = half;
  const ThrPair<R> thr = thr_two_simplex<R>(pos, neg, c);
  Applier<Data> fp(thr.a, kMapIdentity, 1.0), fn(thr.b, kMapIdentity, 1.0);
  for (int j = lane_id(); j < m; j += kLanes) {
    const bool label = (mask[j >> 5] >> (j & 31)) & 1u;
    a[j] = label ? fp(static_cast<Data>(half - v[j])) : -fn(static_cast<Data>(half + v[j]));
  }
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
}

// l2_entropy_topk.h:46-71: v = scores - norm2 * a, v_j -= v_y, x = prox_topk_entropy_biased(v, k,
// alpha = c * norm2), a_y = c * min(1, <1,x>), a_j = -c * x_j.
template <typename R, typename Data>
SDCAB_D void update_dual_variables_entropy_topk(const ObjectiveParams& o, Data norm2,
                                                const Data* scores, Data* a, Data* v, int m, int y) {
  const R c = static_cast<R>(o.c);
  for (int j = lane_id(); j < m; j += kLanes) v[j] = add_rn_(mul_rn_(-norm2, a[j]), scores[j]);
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  const Data shift = -v[y];
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  for (int j = lane_id(); j < m; j += kLanes)
    if (j != y) v[j] += shift;
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  const R alpha = c * static_cast<R>(norm2);
  ShiftedRow<Data> row(v, m, y, Data(0));
  const Thr<R> thr = thr_topk_entropy_biased<R>(row, o.k, alpha);
  Applier<Data> f(thr, kMapScaledLambert, static_cast<double>(alpha));
  const Data minus_c = static_cast<Data>(-c);
  R sum = 0;
  for (int j = lane_id(); j < m; j += kLanes) {
    if (j != y) {
      const Data p = f(v[j]);
      sum += static_cast<R>(p);
      a[j] = minus_c * p;
    }
  }
  sum = warp_sum(sum);
  if (lane_id() == 0) a[y] = static_cast<Data>(c * min_(R(1), sum));
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
}

// scores[0, m): A K_i (or W'x_i); a[0, m): dual variables of the example, updated
// in place; v[0, m): scratch in the same memory space; y: label; norm2 = K_ii.
template <typename R, typename Data>
SDCAB_D void update_dual_variables_multiclass(const ObjectiveParams& o, Data norm2,
                                              const Data* scores, Data* a, Data* v, int m, int y) {
  if (o.id == kObjL2EntropyTopk) {
    update_dual_variables_entropy_topk<R, Data>(o, norm2, scores, a, v, m, y);
    return;
  }
  if (o.id == kObjL2Entropy) {
    update_dual_variables_entropy<R, Data>(o, norm2, scores, a, v, m, y);
    return;
  }
  const R c = static_cast<R>(o.c);
  const bool smooth = (o.id == kObjL2HingeTopkSmooth || o.id == kObjL2TopkHingeSmooth);
  const R rho = smooth ? static_cast<R>(norm2) / (static_cast<R>(norm2) + static_cast<R>(o.gamma) / c)
                       : R(1);
  // 1. v = alpha * scores + beta * a  (beta applied first, then the axpy; two roundings)
  const Data alpha = smooth ? static_cast<Data>(rho) / norm2 : Data(1) / norm2;
  const Data beta = smooth ? -static_cast<Data>(rho) : Data(-1);
  for (int j = lane_id(); j < m; j += kLanes) {
    v[j] = add_rn_(mul_rn_(beta, a[j]), mul_rn_(alpha, scores[j]));
  }
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  const Data shift = alpha - v[y];
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  for (int j = lane_id(); j < m; j += kLanes)
    if (j != y) v[j] += shift;
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
  // 2. proximal step on the m - 1 entries other than the label
  ShiftedRow<Data> row(v, m, y, Data(0));
  Thr<R> thr;
  if (o.id == kObjL2TopkHinge || o.id == kObjL2TopkHingeSmooth) {
    thr = thr_knapsack_le_biased<R>(row, R(0), c / static_cast<R>(o.k), c, rho);
  } else {
    thr = thr_topk_simplex<R>(row, o.k, c, rho);
  }
  Applier<Data> f(thr, kMapIdentity, 1.0);
  R sum = 0;
  for (int j = lane_id(); j < m; j += kLanes) {
    if (j != y) {
      const Data p = f(v[j]);
      sum += static_cast<R>(p);
      a[j] = -p;
    }
  }
  sum = warp_sum(sum);
  // 3. the label's variable
  if (lane_id() == 0) a[y] = static_cast<Data>(min_(c, sum));
#if defined(__CUDA_ARCH__)
  __syncwarp();
#endif
}

}  // namespace sdcab
