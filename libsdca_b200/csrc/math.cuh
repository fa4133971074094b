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

// (1 + x/1024)^1024 by ten squarings   (reference: math/lambert.h:53-62)
template <typename T>
SDCAB_HD T exp_crude(T x) {
  T y = T(1) + x / T(1024);
#pragma unroll
  for (int i = 0; i < 10; ++i) y *= y;
  return y;
}

// W(exp(x)), float table                (reference: math/lambert.h:77-106)
SDCAB_HD float lambert_w_exp(float x) {
  float w;
  if (x > -1.0f) {
    if (x <= 8.0f) {
      w = householder5(x, 1.0f);
    } else {
      return (x <= 536870912.0f) ? householder5(x - log_(x), x) : x;
    }
  } else {
    if (x > -18.0f) {
      w = exp_crude(x);
    } else {
      return (x > -104.0f) ? exp_(x) : 0.0f;
    }
  }
  return householder5(w, exp_(x - w));
}

// W(exp(x)), double table               (reference: math/lambert.h:121-157)
SDCAB_HD double lambert_w_exp(double x) {
  double w;
  if (x > 0.0) {
    if (x <= 4.0) {
      w = householder5(x, 1.0);
    } else if (x <= 576460752303423488.0) {
      w = householder5(x - log_(x), x);
    } else {
      return x;
    }
  } else {
    if (x > -36.0) {
      w = exp_crude(x);
      if (x > -20.0) w = householder5(w, exp_crude(x - w));
    } else {
      return (x > -746.0) ? exp_(x) : 0.0;
    }
  }
  return householder5(w, exp_(x - w));
}

// w + log(w)                             (reference: math/lambert.h:210-214)
template <typename T>
SDCAB_HD T lambert_w_exp_inverse(T w) { return w + log_(w); }

}  // namespace sdcab
