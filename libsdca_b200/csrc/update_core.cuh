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

SDCAB_HD bool objective_has_update(int id) {
  return id == kObjL2HingeTopk || id == kObjL2HingeTopkSmooth || id == kObjL2TopkHinge ||
         id == kObjL2TopkHingeSmooth || id == kObjL2EntropyTopk;
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
