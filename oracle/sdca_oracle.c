/*
 * Test infrastructure: a plain-C restatement of the reference's CPU algorithms
 * for the batched proximal operators, the objective / duality-gap evaluation
 * and the SDCA solver around them (mlapin/libsdca: include/sdca/prox,
 * include/sdca/math, include/sdca/solver/eval*, include/sdca/solver/objective,
 * include/sdca/solver/update.h, include/sdca/solver.h).  The body is
 * sdca_oracle_impl.inc, compiled here for float/double data and float/double
 * accumulators; each function there cites the file:line it follows.
 *
 * Parity of this restatement is pinned by tests/test_oracle_restatement.py,
 * which checks it against the reference's own headers (oracle/_ref) on the
 * regimes of the reference's tests, and against the committed golden vectors.
 *
 * Only tests, the smoke check and bench.py's CPU-baseline legs may call this;
 * the product library never does.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  double lo, hi, rhs, rho, alpha;
  int64_t k, p;
} oracle_opts;

typedef struct {
  int objective;
  double c, gamma;
  int64_t k;
  int input_kind;
  int64_t d, n, m;
  const void* X;
  void* A;
  void* W;
  const void* W0;
  const int64_t* labels;
  const int64_t* offsets;
  int is_train;
  int nthreads;
  double epsilon;
  int64_t max_epoch, eval_epoch;
  int eval_on_start;
} oracle_eval_args;

#define CAT2(a, b) a##_##b
#define CAT(a, b) CAT2(a, b)

/* float data, float accumulators */
#define D float
#define D_EPS FLT_EPSILON
#define R float
#define FN(x) CAT(x, ff)
#define R_EPS FLT_EPSILON
#define R_MIN FLT_MIN
#define R_MAX FLT_MAX
#define R_EXP_MIN_ARG (-8.733654022216796875000000e+01f) /* math/log_exp.h:47-52 */
#define R_EXP expf
#define R_LOG logf
#define R_LOG1P log1pf
#define R_FABS fabsf
#define R_LAMBERT lambert_w_exp_f
#define D_EXP expf
#define D_LAMBERT lambert_w_exp_f
#include "sdca_oracle_impl.inc"
#undef D
#undef R
#undef FN
#undef R_EPS
#undef R_MIN
#undef R_MAX
#undef D_EPS
#undef R_EXP_MIN_ARG
#undef R_EXP
#undef R_LOG
#undef R_LOG1P
#undef R_FABS
#undef R_LAMBERT
#undef D_EXP
#undef D_LAMBERT

/* float data, double accumulators (the reference's default for float input) */
#define D float
#define D_EPS FLT_EPSILON
#define R double
#define FN(x) CAT(x, fd)
#define R_EPS DBL_EPSILON
#define R_MIN DBL_MIN
#define R_MAX DBL_MAX
#define R_EXP_MIN_ARG (log(DBL_MIN)) /* math/log_exp.h:33-35 */
#define R_EXP exp
#define R_LOG log
#define R_LOG1P log1p
#define R_FABS fabs
#define R_LAMBERT lambert_w_exp_d
#define D_EXP expf
#define D_LAMBERT lambert_w_exp_f
#include "sdca_oracle_impl.inc"
#undef D
#undef R
#undef FN
#undef R_EPS
#undef R_MIN
#undef R_MAX
#undef D_EPS
#undef R_EXP_MIN_ARG
#undef R_EXP
#undef R_LOG
#undef R_LOG1P
#undef R_FABS
#undef R_LAMBERT
#undef D_EXP
#undef D_LAMBERT

/* double data, float accumulators */
#define D double
#define D_EPS DBL_EPSILON
#define R float
#define FN(x) CAT(x, df)
#define R_EPS FLT_EPSILON
#define R_MIN FLT_MIN
#define R_MAX FLT_MAX
#define R_EXP_MIN_ARG (-8.733654022216796875000000e+01f)
#define R_EXP expf
#define R_LOG logf
#define R_LOG1P log1pf
#define R_FABS fabsf
#define R_LAMBERT lambert_w_exp_f
#define D_EXP exp
#define D_LAMBERT lambert_w_exp_d
#include "sdca_oracle_impl.inc"
#undef D
#undef R
#undef FN
#undef R_EPS
#undef R_MIN
#undef R_MAX
#undef D_EPS
#undef R_EXP_MIN_ARG
#undef R_EXP
#undef R_LOG
#undef R_LOG1P
#undef R_FABS
#undef R_LAMBERT
#undef D_EXP
#undef D_LAMBERT

/* double data, double accumulators */
#define D double
#define D_EPS DBL_EPSILON
#define R double
#define FN(x) CAT(x, dd)
#define R_EPS DBL_EPSILON
#define R_MIN DBL_MIN
#define R_MAX DBL_MAX
#define R_EXP_MIN_ARG (log(DBL_MIN))
#define R_EXP exp
#define R_LOG log
#define R_LOG1P log1p
#define R_FABS fabs
#define R_LAMBERT lambert_w_exp_d
#define D_EXP exp
#define D_LAMBERT lambert_w_exp_d
#include "sdca_oracle_impl.inc"

/* dtype / result: 0 = float, 1 = double (same convention as oracle/ref_shim.cpp) */
int sdca_oracle_prox(const char* prox, int dtype, int result, void* a, int64_t m, int64_t n,
                     const oracle_opts* o, int nthreads) {
  (void)nthreads;
  if (dtype == 0 && result == 0) return run_ff(prox, (float*)a, m, n, o, 0, 0, 0, 0, 0, 1);
  if (dtype == 0 && result == 1) return run_fd(prox, (float*)a, m, n, o, 0, 0, 0, 0, 0, 1);
  if (dtype == 1 && result == 0) return run_df(prox, (double*)a, m, n, o, 0, 0, 0, 0, 0, 1);
  if (dtype == 1 && result == 1) return run_dd(prox, (double*)a, m, n, o, 0, 0, 0, 0, 0, 1);
  return -2;
}

int sdca_oracle_thresholds(const char* prox, int dtype, int result, const void* a, int64_t m,
                           int64_t n, const oracle_opts* o, double* t, double* lo, double* hi,
                           int64_t* nU, int64_t* nM) {
  if (dtype == 0 && result == 0) return run_ff(prox, (float*)a, m, n, o, t, lo, hi, nU, nM, 0);
  if (dtype == 0 && result == 1) return run_fd(prox, (float*)a, m, n, o, t, lo, hi, nU, nM, 0);
  if (dtype == 1 && result == 0) return run_df(prox, (double*)a, m, n, o, t, lo, hi, nU, nM, 0);
  if (dtype == 1 && result == 1) return run_dd(prox, (double*)a, m, n, o, t, lo, hi, nU, nM, 0);
  return -2;
}

/* Rows on which the reference's two_simplex_sort (prox/two_simplex_sort.h:84-97) stays inside its
 * arrays; on the others it reads past the end of a block and has no defined result. */
int sdca_oracle_two_simplex_sort_defined(int dtype, int result, const void* a, int64_t m, int64_t n,
                                         int64_t p, double rhs, int32_t* defined) {
  if (p < 1 || p > m - 1) return -3;
  if (dtype == 0 && result == 0) return two_simplex_sort_defined_ff((const float*)a, m, n, p, (float)rhs, defined);
  if (dtype == 0 && result == 1) return two_simplex_sort_defined_fd((const float*)a, m, n, p, rhs, defined);
  if (dtype == 1 && result == 0) return two_simplex_sort_defined_df((const double*)a, m, n, p, (float)rhs, defined);
  if (dtype == 1 && result == 1) return two_simplex_sort_defined_dd((const double*)a, m, n, p, rhs, defined);
  return -2;
}

int sdca_oracle_eval(const oracle_eval_args* a, int dtype, int result, double* out, double* acc) {
  if (dtype == 0 && result == 0) return eval_ff(a, out, acc);
  if (dtype == 0 && result == 1) return eval_fd(a, out, acc);
  if (dtype == 1 && result == 0) return eval_df(a, out, acc);
  if (dtype == 1 && result == 1) return eval_dd(a, out, acc);
  return -2;
}

/* The example order of every epoch of the reference's solver (include/sdca/solver.h:59,
 * 77-79,96-100): a default-seeded std::minstd_rand (x <- 48271 x mod 2^31 - 1 from 1)
 * driving std::shuffle as libstdc++ implements it, on one index vector kept across epochs. */
static uint64_t minstd_next(uint64_t* x) { *x = (*x * 48271ull) % 2147483647ull; return *x; }
static uint64_t uniform_upto(uint64_t* g, uint64_t hi) {
  const uint64_t grange = 2147483646ull - 1ull;
  uint64_t ret;
  if (grange > hi) {
    const uint64_t span = hi + 1, scaling = grange / span, past = span * scaling;
    do { ret = minstd_next(g) - 1; } while (ret >= past);
    ret /= scaling;
  } else if (grange < hi) {
    const uint64_t gspan = grange + 1;
    uint64_t tmp;
    do {
      tmp = gspan * uniform_upto(g, hi / gspan);
      ret = tmp + (minstd_next(g) - 1);
    } while (ret > hi || ret < tmp);
  } else {
    ret = minstd_next(g) - 1;
  }
  return ret;
}
int sdca_oracle_epoch_permutations(int64_t n, int64_t num_epochs, int64_t* perm) {
  uint64_t g = 1;
  int64_t* v = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n > 0 ? n : 1));
  if (!v) return -9;
  for (int64_t i = 0; i < n; ++i) v[i] = i;
  const uint64_t grange = 2147483646ull - 1ull;
  for (int64_t e = 0; e < num_epochs; ++e) {
    const uint64_t un = (uint64_t)n;
    if (un > 0 && grange / un >= un) {        /* two positions per draw */
      uint64_t i = 1;
      if (un % 2 == 0 && un > 1) { uint64_t j = uniform_upto(&g, 1); int64_t t = v[i]; v[i] = v[j]; v[j] = t; ++i; }
      while (i < un) {
        const uint64_t b0 = i + 1, b1 = b0 + 1;
        const uint64_t x = uniform_upto(&g, b0 * b1 - 1);
        uint64_t j = x / b1; int64_t t = v[i]; v[i] = v[j]; v[j] = t; ++i;
        j = x % b1; t = v[i]; v[i] = v[j]; v[j] = t; ++i;
      }
    } else {
      for (uint64_t i = 1; i < un; ++i) { uint64_t j = uniform_upto(&g, i); int64_t t = v[i]; v[i] = v[j]; v[j] = t; }
    }
    for (int64_t i = 0; i < n; ++i) perm[e * n + i] = v[i];
  }
  free(v);
  return 0;
}

int sdca_oracle_fit(const oracle_eval_args* a, int dtype, int result, double* hist, int64_t hist_cap,
                    int64_t* num_evals, int64_t* epoch, int* status, double* acc_last) {
  if (a->max_epoch < 0 || a->n <= 0) return -2;
  int64_t epochs = a->max_epoch > 0 ? a->max_epoch : 1;
  int64_t* perm = (int64_t*)malloc(sizeof(int64_t) * (size_t)(epochs * a->n));
  if (!perm) return -9;
  int rc = sdca_oracle_epoch_permutations(a->n, epochs, perm);
  if (rc == 0) {
    if (dtype == 0 && result == 0) rc = fit_ff(a, perm, hist, hist_cap, num_evals, epoch, status, acc_last);
    else if (dtype == 0 && result == 1) rc = fit_fd(a, perm, hist, hist_cap, num_evals, epoch, status, acc_last);
    else if (dtype == 1 && result == 0) rc = fit_df(a, perm, hist, hist_cap, num_evals, epoch, status, acc_last);
    else if (dtype == 1 && result == 1) rc = fit_dd(a, perm, hist, hist_cap, num_evals, epoch, status, acc_last);
    else rc = -2;
  }
  free(perm);
  return rc;
}

double sdca_oracle_lambert_w_exp_f64(double x) { return lambert_w_exp_d(x); }
float sdca_oracle_lambert_w_exp_f32(float x) { return lambert_w_exp_f(x); }
