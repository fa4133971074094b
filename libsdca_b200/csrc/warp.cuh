// Warp-cooperative building blocks shared by every row kernel.
//
// One group of lanes owns one row (one vector of the N x m matrix).  All lanes
// of the group execute the same control flow; data-dependent decisions are
// taken on values that a butterfly reduction has made identical in every lane.
//
// The same templates also compile for the host with a group of exactly one
// lane (SDCAB_HOST_SINGLE_LANE), where every reduction is the identity.  That
// build exists only so the CPU test-suite can exercise the threshold logic
// without a GPU; it is not a product path and is never linked into the library.
#pragma once

#include <cfloat>
#include <cmath>
#include <cstdint>

#if defined(__CUDACC__)
#define SDCAB_HD __host__ __device__ __forceinline__
#define SDCAB_D __device__ __forceinline__
#else
#define SDCAB_HD inline
#define SDCAB_D inline
#endif

namespace sdcab {

#if defined(__CUDA_ARCH__)
constexpr int kLanes = 32;
SDCAB_D int lane_id() { return static_cast<int>(threadIdx.x) & 31; }
#else
constexpr int kLanes = 1;
SDCAB_D int lane_id() { return 0; }
#endif

constexpr unsigned kFullMask = 0xffffffffu;

// ---- butterfly reductions: every lane receives the result -----------------
template <typename T>
SDCAB_D T shfl_xor(T v, int mask) {
#if defined(__CUDA_ARCH__)
  return __shfl_xor_sync(kFullMask, v, mask);
#else
  (void)mask;
  return v;
#endif
}

template <typename T>
SDCAB_D T shfl_idx(T v, int src) {
#if defined(__CUDA_ARCH__)
  return __shfl_sync(kFullMask, v, src);
#else
  (void)src;
  return v;
#endif
}

template <typename T>
SDCAB_D T warp_sum(T v) {
#if defined(__CUDA_ARCH__)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
#endif
  return v;
}

// integer sums and maxima are single redux.sync instructions
SDCAB_D int warp_sum(int v) {
#if defined(__CUDA_ARCH__)
  return __reduce_add_sync(kFullMask, v);
#else
  return v;
#endif
}

template <typename T>
SDCAB_D T warp_max(T v) {
#if defined(__CUDA_ARCH__)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    T w = __shfl_xor_sync(kFullMask, v, o);
    v = (w > v) ? w : v;
  }
#endif
  return v;
}

template <typename T>
SDCAB_D T warp_min(T v) {
#if defined(__CUDA_ARCH__)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    T w = __shfl_xor_sync(kFullMask, v, o);
    v = (w < v) ? w : v;
  }
#endif
  return v;
}

// Largest value together with the smallest index that holds it.
template <typename T>
SDCAB_D void warp_argmax(T& v, int& idx) {
#if defined(__CUDA_ARCH__)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    T w = __shfl_xor_sync(kFullMask, v, o);
    int j = __shfl_xor_sync(kFullMask, idx, o);
    if (w > v || (w == v && j < idx)) { v = w; idx = j; }
  }
#else
  (void)v; (void)idx;
#endif
}

// ---- numeric traits --------------------------------------------------------
template <typename T> struct num;
template <> struct num<float> {
  static SDCAB_HD float eps() { return FLT_EPSILON; }
  static SDCAB_HD float tiny() { return FLT_MIN; }
  static SDCAB_HD float inf() { return INFINITY; }
  static SDCAB_HD float max() { return FLT_MAX; }
  // smallest argument whose exponential is a normal number
  // (the reference pins these for float, include/sdca/math/log_exp.h:47-52)
  static SDCAB_HD float exp_min_arg() { return -8.733654022216796875000000e+01f; }
};
template <> struct num<double> {
  static SDCAB_HD double eps() { return DBL_EPSILON; }
  static SDCAB_HD double tiny() { return DBL_MIN; }
  static SDCAB_HD double inf() { return static_cast<double>(INFINITY); }
  static SDCAB_HD double max() { return DBL_MAX; }
  // log(DBL_MIN), the value std::log(std::numeric_limits<double>::min()) takes
  // (include/sdca/math/log_exp.h:33-35)
  static SDCAB_HD double exp_min_arg() { return -7.083964185322641e+02; }
};

SDCAB_HD float exp_(float x) { return ::expf(x); }
SDCAB_HD double exp_(double x) { return ::exp(x); }
SDCAB_HD float log_(float x) { return ::logf(x); }
SDCAB_HD double log_(double x) { return ::log(x); }
SDCAB_HD float log1p_(float x) { return ::log1pf(x); }
SDCAB_HD double log1p_(double x) { return ::log1p(x); }
SDCAB_HD float abs_(float x) { return ::fabsf(x); }
SDCAB_HD double abs_(double x) { return ::fabs(x); }
template <typename T> SDCAB_HD T max_(T a, T b) { return (a < b) ? b : a; }
template <typename T> SDCAB_HD T min_(T a, T b) { return (b < a) ? b : a; }
SDCAB_HD bool finite_(float x) { return ::fabsf(x) <= FLT_MAX; }
SDCAB_HD bool finite_(double x) { return ::fabs(x) <= DBL_MAX; }

}  // namespace sdcab
