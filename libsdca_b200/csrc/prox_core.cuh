// Dispatch from an operator id to its threshold routine, and the elementwise
// step  x <- max(lo, min(map(x - t), hi))  that every operator ends with
// (include/sdca/prox/proxdef.h:164-196 of the reference: the thresholds are
// cast to the data type first, then the map and the clip run in data precision).
#pragma once

#include "thresholds.cuh"

namespace sdcab {

enum ProxId {
  kKnapsackEq = 0,
  kKnapsackLe,
  kKnapsackLeBiased,
  kTopkSimplex,
  kTopkSimplexBiased,
  kTopkCone,
  kTopkConeBiased,
  kEntropy,
  kEntropyNorm,
  kTopkEntropy,
  kTopkEntropyBiased,
  kTwoSimplex,
  kTwoSimplexSort,
  kLambertWExp,
  kNumProx
};

enum MapId { kMapIdentity = 0, kMapExp, kMapLambert, kMapScaledLambert };

struct ProxParams {
  double lo, hi, rhs, rho, alpha;
  int k, p;
  int accurate;   // exact recomputation of t after variable fixing (SDCA_ACCURATE_MATH)
};

SDCAB_HD MapId prox_map(int prox) {
  switch (prox) {
    case kEntropy: case kTopkEntropy: return kMapExp;
    case kEntropyNorm: return kMapLambert;
    case kTopkEntropyBiased: return kMapScaledLambert;
    default: return kMapIdentity;
  }
}

template <typename R, typename Row>
SDCAB_D Thr<R> compute_thresholds(int prox, const Row& row, const ProxParams& q) {
  const R lo = static_cast<R>(q.lo), hi = static_cast<R>(q.hi);
  const R rhs = static_cast<R>(q.rhs), rho = static_cast<R>(q.rho);
  switch (prox) {
    case kKnapsackEq: return thr_knapsack_eq<R>(row, lo, hi, rhs, q.accurate != 0);
    case kKnapsackLe: return thr_knapsack_le<R>(row, lo, hi, rhs, q.accurate != 0);
    case kKnapsackLeBiased: return thr_knapsack_le_biased<R>(row, lo, hi, rhs, rho, q.accurate != 0);
    case kTopkSimplex: return thr_topk_simplex<R>(row, q.k, rhs, R(0), q.accurate != 0);
    case kTopkSimplexBiased: return thr_topk_simplex<R>(row, q.k, rhs, rho, q.accurate != 0);
    case kTopkCone: return thr_topk_cone<R>(row, q.k, R(0));
    case kTopkConeBiased: return thr_topk_cone<R>(row, q.k, rho);
    case kEntropy: return thr_entropy<R>(row, hi, rhs);
    case kEntropyNorm: return thr_entropy_norm<R>(row, hi, rhs);
    case kTopkEntropy: return thr_topk_entropy<R>(row, q.k);
    case kTopkEntropyBiased:
      return thr_topk_entropy_biased<R>(row, q.k, static_cast<R>(q.alpha));
    default: break;
  }
  return make_thr(R(0), R(0), R(0), 0, 0, R(0), R(0));
}

// Status of a row as the thresholds entry points report it.
template <typename R>
SDCAB_HD int thr_status(const Thr<R>& t) {
  return t.status | ((finite_(t.t) && finite_(t.hi) && finite_(t.lo)) ? 0 : kThrNotFinite);
}

// The clip of proxdef.h:176-177 with std::max / std::min operand order.
template <typename Data>
SDCAB_HD Data clip_(Data v, Data lo, Data hi) {
  const Data w = (hi < v) ? hi : v;
  return (lo < w) ? w : lo;
}

template <typename Data>
struct Applier {
  Data t, lo, hi, scale;
  int map;
  template <typename R>
  SDCAB_HD Applier(const Thr<R>& thr, int map_, double alpha)
      : t(static_cast<Data>(thr.t)), lo(static_cast<Data>(thr.lo)),
        hi(static_cast<Data>(thr.hi)),
        scale(Data(1) / static_cast<Data>(alpha)), map(map_) {}
  SDCAB_HD Data operator()(Data x) const {
    Data v = x - t;
    switch (map) {
      case kMapExp: v = exp_(v); break;
      case kMapLambert: v = lambert_w_exp(v); break;
      case kMapScaledLambert: v = scale * lambert_w_exp(v); break;
      default: break;
    }
    return clip_(v, lo, hi);
  }
};

}  // namespace sdcab
