// Scalar math of the proximal operators: Lambert W of exp(x), x*log(x).
//
// Behaviour follows include/sdca/math/lambert.h and include/sdca/math/log_exp.h
// of the reference: the same interval table, the same crude exponential seed
// and the same number of fifth-order Householder steps, because for moderate
// negative arguments the seed and the step count are part of the result.
#pragma once

#include "warp.cuh"

namespace sdcab {

// x * log(x), 0 for x <= 0            (reference: math/log_exp.h:76-80)
template <typename T>
SDCAB_HD T x_log_x(T x) { return (x > 0) ? x * log_(x) : T(0); }

// One fifth-order Householder step for w - z*exp(-w) = 0 with y = z*exp(-w).
// (reference: math/lambert.h:31-42)
template <typename T>
SDCAB_HD T householder5(T w, T y) {
  const T f0 = w - y, f1 = T(1) + y;
  const T f11 = f1 * f1, f0y = f0 * y;
  const T f00y = f0 * f0y;
  return w - T(4) * f0 * (T(6) * f1 * (f11 + f0y) + f00y) /
                 (f11 * (T(24) * f11 + T(36) * f0y) + f00y * (T(14) * y + f0 + T(8)));
}

#if defined(__CUDA_ARCH__)
// The same step for float data on the device with the quotient formed by the fast
// division (reciprocal approximation and a multiply, 2 ulp): the quotient is the
// correction term of a fifth-order step, a few per cent of w at most, so its last bits
// do not reach the result, and an IEEE division costs as much as the rest of the step.
__device__ __forceinline__ float householder5_fast(float w, float y) {
  const float f0 = w - y, f1 = 1.0f + y;
  const float f11 = f1 * f1, f0y = f0 * y;
  const float f00y = f0 * f0y;
  return w - __fdividef(4.0f * f0 * (6.0f * f1 * (f11 + f0y) + f00y),
                        f11 * (24.0f * f11 + 36.0f * f0y) + f00y * (14.0f * y + f0 + 8.0f));
}
#endif

// (1 + x/1024)^1024 by ten squarings   (reference: math/lambert.h:53-62)
template <typename T>
SDCAB_HD T exp_crude(T x) {
  T y = T(1) + x / T(1024);
#pragma unroll
  for (int i = 0; i < 10; ++i) y *= y;
  return y;
}

// W(exp(x)), float table                (reference: math/lambert.h:77-106)
//   (-inf, -104] -> 0           (-104, -18] -> exp(x)
//   (-18, -1]    -> one step from the crude exponential
//   (-1, 8]      -> two steps from w = x
//   (8, 2^29]    -> one step from x - log(x) with y = x        above -> x
// Written without divergent branches: the lanes of a warp usually fall into
// several intervals, so both seeds are computed and the operands of the one
// exponential and of the final step are selected; each interval still sees
// exactly the operations the table prescribes for it.
SDCAB_HD float lambert_w_exp(float x) {
  const bool upper = x > -1.0f;                 // (-1, +inf)
  const bool tail_lo = !(x > -18.0f);           // (-inf, -18]
  const bool tail_hi = x > 8.0f;                // (8, +inf)
#if defined(__CUDA_ARCH__)
  const float seed = upper ? householder5_fast(x, 1.0f) : exp_crude(x);
#else
  const float seed = upper ? householder5(x, 1.0f) : exp_crude(x);
#endif
  const float e = exp_(tail_lo ? x : x - seed);
#if defined(__CUDA_ARCH__)
  // x > 8: the seed x - log(x) feeds one fifth-order step; the fast logarithm's absolute
  // error of 2e-7 on a seed of 6 and more is far below what that step removes
  const float w_in = tail_hi ? x - __logf(x) : seed;
#else
  const float w_in = tail_hi ? x - log_(x) : seed;
#endif
  const float y_in = tail_hi ? x : e;
#if defined(__CUDA_ARCH__)
  const float stepped = householder5_fast(w_in, y_in);
#else
  const float stepped = householder5(w_in, y_in);
#endif
  if (tail_lo) return (x > -104.0f) ? e : 0.0f;
  if (tail_hi && !(x <= 536870912.0f)) return x;
  return stepped;
}

// W(exp(x)), double table               (reference: math/lambert.h:121-157)
//   (-inf, -746] -> 0            (-746, -36] -> exp(x)
//   (-36, -20]   -> one step from the crude exponential
//   (-20, 0]     -> crude seed, one step with the crude exponential, one step
//   (0, 4]       -> two steps from w = x
//   (4, 2^59]    -> step from x - log(x) with y = x, then one step   above -> x
SDCAB_HD double lambert_w_exp(double x) {
  const bool pos = x > 0.0;
  const bool tail_lo = !(x > -36.0);
  const bool tail_hi = x > 4.0;
  double w;
  if (pos) {
    w = tail_hi ? householder5(x - log_(x), x) : householder5(x, 1.0);
  } else {
    w = exp_crude(x);
    if (x > -20.0) w = householder5(w, exp_crude(x - w));
  }
  const double e = exp_(tail_lo ? x : x - w);
  if (tail_lo) return (x > -746.0) ? e : 0.0;
  if (tail_hi && !(x <= 576460752303423488.0)) return x;
  return householder5(w, e);
}

// w + log(w)                             (reference: math/lambert.h:210-214)
template <typename T>
SDCAB_HD T lambert_w_exp_inverse(T w) { return w + log_(w); }

}  // namespace sdcab
