// Host-side pieces of the fit: the example order of every epoch and the
// stopping rule.  Plain C++, no CUDA, so the CPU tests can use them directly.
#pragma once

#include <cmath>
#include <cstdint>
#include <limits>
#include <vector>

#include "../../include/sdca_b200.h"

namespace sdcab {

// std::minstd_rand: x <- 48271 x mod (2^31 - 1), default seed 1, values in
// [1, 2^31 - 2].
struct MinstdRand {
  uint64_t x = 1;
  static constexpr uint64_t kMin = 1, kMax = 2147483646ull;
  uint64_t operator()() { x = (x * 48271ull) % 2147483647ull; return x; }
};

// A uniform integer in [0, hi] drawn the way libstdc++'s
// std::uniform_int_distribution<unsigned long> draws it from a generator whose
// range is not a power of two: rejection on a scaled range when the generator
// covers it, digits in base (range + 1) otherwise.
inline uint64_t uniform_upto(MinstdRand& g, uint64_t hi) {
  const uint64_t grange = MinstdRand::kMax - MinstdRand::kMin;
  uint64_t ret;
  if (grange > hi) {
    const uint64_t span = hi + 1;
    const uint64_t scaling = grange / span;
    const uint64_t past = span * scaling;
    do { ret = g() - MinstdRand::kMin; } while (ret >= past);
    ret /= scaling;
  } else if (grange < hi) {
    const uint64_t gspan = grange + 1;
    uint64_t tmp;
    do {
      tmp = gspan * uniform_upto(g, hi / gspan);
      ret = tmp + (g() - MinstdRand::kMin);
    } while (ret > hi || ret < tmp);
  } else {
    ret = g() - MinstdRand::kMin;
  }
  return ret;
}

// std::shuffle of libstdc++ (bits/stl_algo.h, GCC 7 and later): when the
// generator's range covers n^2, two swap positions come out of one draw; else
// one draw per position.  The reference's solver applies it to the same index
// vector at the start of every epoch (include/sdca/solver.h:77-79,96-100), so
// the order of epoch e depends on all earlier epochs.
inline void shuffle_like_libstdcxx(std::vector<int64_t>& v, MinstdRand& g) {
  const uint64_t n = v.size();
  if (n == 0) return;
  const uint64_t grange = MinstdRand::kMax - MinstdRand::kMin;
  auto swap_at = [&](uint64_t i, uint64_t j) { int64_t t = v[i]; v[i] = v[j]; v[j] = t; };
  if (grange / n >= n) {
    uint64_t i = 1;
    if ((n % 2) == 0) { swap_at(i, uniform_upto(g, 1)); ++i; }
    while (i != n) {
      const uint64_t b0 = i + 1, b1 = b0 + 1;
      const uint64_t x = uniform_upto(g, b0 * b1 - 1);
      swap_at(i, x / b1); ++i;
      swap_at(i, x % b1); ++i;
    }
    return;
  }
  for (uint64_t i = 1; i != n; ++i) swap_at(i, uniform_upto(g, i));
}

// The order of `num_epochs` consecutive epochs, perm[e * n + s] = the example
// visited at step s of epoch e.
inline void epoch_permutations(int64_t n, int64_t num_epochs, int64_t* perm) {
  MinstdRand g;
  std::vector<int64_t> v(static_cast<size_t>(n));
  for (int64_t i = 0; i < n; ++i) v[static_cast<size_t>(i)] = i;
  for (int64_t e = 0; e < num_epochs; ++e) {
    shuffle_like_libstdcxx(v, g);
    for (int64_t i = 0; i < n; ++i) perm[e * n + i] = v[static_cast<size_t>(i)];
  }
}

// check_stopping_criteria of the reference (include/sdca/solver/eval.h:56-109):
// `last` / `before` are the two most recent evaluations of the training set
// (either may be null); cpu_now / wall_now are the seconds spent so far, compared
// with the limits when those are positive.  Returns the new status.
inline int check_stopping(int status, const sdcab_eval_record* last,
                          const sdcab_eval_record* before, double epsilon, int64_t epoch,
                          int64_t max_epoch, double data_epsilon, double max_cpu_time = 0,
                          double cpu_now = 0, double max_wall_time = 0, double wall_now = 0) {
  if (status != SDCAB_FIT_SOLVING) return status;
  if (last) {
    const double gap = last->primal - last->dual;
    const double mx = std::fmax(std::fabs(last->primal), std::fabs(last->dual));
    const double eps_stop = mx * epsilon;
    const double eps = 64 * std::fmax(1.0, mx) *
                       std::fmax(std::numeric_limits<double>::epsilon(), data_epsilon);
    if (gap < eps_stop) {
      status = (gap < -eps || gap <= -eps_stop) ? SDCAB_FIT_FAILED : SDCAB_FIT_SOLVED;
    } else if (before) {
      if (last->dual + eps * std::fabs(before->dual) < before->dual) status = SDCAB_FIT_NO_PROGRESS;
    }
  }
  if (status == SDCAB_FIT_SOLVING) {
    if (epoch >= max_epoch) status = SDCAB_FIT_MAX_EPOCH;
    else if (max_cpu_time > 0 && cpu_now >= max_cpu_time) status = SDCAB_FIT_MAX_CPU_TIME;
    else if (max_wall_time > 0 && wall_now >= max_wall_time) status = SDCAB_FIT_MAX_WALL_TIME;
  }
  return status;
}

}  // namespace sdcab
