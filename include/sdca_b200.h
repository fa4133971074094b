/*
 * sdca_b200 -- C ABI of the B200 (sm_100a) implementation of libsdca's
 * data-parallel hot path: batched proximal operators and the solver's
 * objective / duality-gap evaluation.
 *
 * Plain pointers and sizes only.  Every entry point returns SDCAB_OK (0) or a
 * negative sdcab_status and never aborts.  Pointers named *_dev must be device
 * memory of the current CUDA device; `stream` is a cudaStream_t passed as
 * void* (NULL = the default stream).  Host entry points (no _dev suffix) copy
 * their operands to the device and back themselves.
 *
 * There is no CPU fallback: without a usable CUDA device the entry points
 * return SDCAB_ERR_NO_DEVICE / SDCAB_ERR_CUDA.
 *
 * Matrix layout: the reference's Matlab front end passes an m x N column-major
 * array whose columns are the vectors; that is the same memory as an N x m
 * row-major matrix, which is how it is described here: row j is the j-th
 * vector, stored at [j*m, (j+1)*m).
 *
 * Citations name files of the reference project (mlapin/libsdca) that each
 * entry point stands in for.
 */
#ifndef SDCA_B200_H
#define SDCA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; the argument errors mirror the LIBSDCA:* identifiers of the
 * reference's Matlab layer (src/matlab/mex_util.h:68-165). */
typedef enum sdcab_status {
  SDCAB_OK = 0,
  SDCAB_ERR_ARG = -1,            /* LIBSDCA:arg             */
  SDCAB_ERR_ARG_RANGE = -2,      /* LIBSDCA:arg_range       */
  SDCAB_ERR_ARG_CLASS = -3,      /* LIBSDCA:arg_class       */
  SDCAB_ERR_NOT_EMPTY = -4,      /* LIBSDCA:arg_not_empty   */
  SDCAB_ERR_LABELS_RANGE = -5,   /* LIBSDCA:labels_range    */
  SDCAB_ERR_PROX = -6,           /* LIBSDCA:prox            */
  SDCAB_ERR_OBJECTIVE = -7,      /* LIBSDCA:objective       */
  SDCAB_ERR_PRECISION = -8,      /* LIBSDCA:precision       */
  SDCAB_ERR_OUT_OF_MEMORY = -9,  /* LIBSDCA:out_of_memory   */
  SDCAB_ERR_NOT_IMPLEMENTED = -10, /* LIBSDCA:not_implemented */
  SDCAB_ERR_NUM_DIM = -11,       /* LIBSDCA:num_dim / num_classes / num_examples */
  SDCAB_ERR_CUDA = -20,
  SDCAB_ERR_NO_DEVICE = -21,
  SDCAB_ERR_TOO_LARGE = -22
} sdcab_status;

const char* sdcab_status_string(int status);
/* Text of the last CUDA error seen by the calling thread ("" if none). */
const char* sdcab_last_error(void);
const char* sdcab_version(void);

/* ---------------------------------------------------------------- prox ---- */

/* Precision of thresholds and accumulators (the reference's Result template
 * parameter; matsdca_prox opts.precision, src/matlab/mex_prox.cpp:189-200).
 * "long double" has no device counterpart and is rejected. */
enum { SDCAB_PRECISION_DOUBLE = 0, SDCAB_PRECISION_FLOAT = 1 };

/* Options of matsdca_prox with the same defaults
 * (src/matlab/mex_prox.cpp:121-127): lo=0 hi=1 rhs=1 rho=1 alpha=1 k=1 p=1. */
typedef struct sdcab_prox_opts {
  double lo, hi, rhs, rho, alpha;
  int64_t k, p;
  int32_t precision;
  int32_t reserved;
} sdcab_prox_opts;

void sdcab_prox_opts_default(sdcab_prox_opts* opts);

/* Per-vector thresholds: prox(a) = max(lo, min(map(a - t), hi)); num_hi and
 * num_mid are the sizes of the sets the reference returns as iterator ranges
 * (include/sdca/prox/proxdef.h:29-67).  For the two-block operators every
 * vector has two consecutive records (first block, second block). */
typedef struct sdcab_thresholds {
  double t, lo, hi;
  int32_t num_hi, num_mid;
} sdcab_thresholds;

/*
 * Batched proximal operator, in place, on n vectors of length m.
 * Replaces prox_<name>(dim, first, last, aux, ...) of include/sdca/prox/<name>.h
 * (batched driver: include/sdca/prox/proxdef.h:279-324) as dispatched by
 * matsdca_prox (src/matlab/mex_prox.cpp:143-176).  `prox` is one of
 *   knapsack | knapsack_eq | knapsack_le | knapsack_le_biased | topk_simplex |
 *   topk_simplex_biased | topk_cone | topk_cone_biased | entropy |
 *   entropy_norm | topk_entropy | topk_entropy_biased | two_simplex |
 *   two_simplex_sort | lambert_w_exp
 * Argument checks are those of src/matlab/mex_prox.cpp:132-136.
 */
int sdcab_prox_f32_dev(const char* prox, float* a_dev, int64_t m, int64_t n,
                       const sdcab_prox_opts* opts, void* stream);
int sdcab_prox_f64_dev(const char* prox, double* a_dev, int64_t m, int64_t n,
                       const sdcab_prox_opts* opts, void* stream);

/* Same, reading a_dev and writing out_dev (matsdca_prox with an output argument
 * duplicates the array first, src/matlab/mex_prox.cpp:113-119); out_dev may
 * equal a_dev. */
int sdcab_prox_to_f32_dev(const char* prox, const float* a_dev, float* out_dev,
                          int64_t m, int64_t n, const sdcab_prox_opts* opts,
                          void* stream);
int sdcab_prox_to_f64_dev(const char* prox, const double* a_dev, double* out_dev,
                          int64_t m, int64_t n, const sdcab_prox_opts* opts,
                          void* stream);

/* Host-buffer form: `a` is read, the result is written to `out` (out == a or
 * out == NULL means in place, like matsdca_prox with no output argument,
 * src/matlab/mex_prox.cpp:113-119).  Synchronous. */
int sdcab_prox_f32(const char* prox, float* a, int64_t m, int64_t n,
                   const sdcab_prox_opts* opts, float* out);
int sdcab_prox_f64(const char* prox, double* a, int64_t m, int64_t n,
                   const sdcab_prox_opts* opts, double* out);

/* Thresholds only (thresholds_<name>(first, last, ...) of each prox header);
 * the data is not modified.  thr_dev holds n records (2n for two-block). */
int sdcab_thresholds_f32_dev(const char* prox, const float* a_dev, int64_t m,
                             int64_t n, const sdcab_prox_opts* opts,
                             sdcab_thresholds* thr_dev, void* stream);
int sdcab_thresholds_f64_dev(const char* prox, const double* a_dev, int64_t m,
                             int64_t n, const sdcab_prox_opts* opts,
                             sdcab_thresholds* thr_dev, void* stream);
int sdcab_thresholds_f32(const char* prox, const float* a, int64_t m, int64_t n,
                         const sdcab_prox_opts* opts, sdcab_thresholds* thr);
int sdcab_thresholds_f64(const char* prox, const double* a, int64_t m, int64_t n,
                         const sdcab_prox_opts* opts, sdcab_thresholds* thr);

/* x <- W(exp(x)) elementwise: apply(dim, first, last, lambert_w_exp_map<Data>())
 * (include/sdca/prox/proxdef.h:386-400, include/sdca/math/lambert.h:77-157). */
int sdcab_lambert_w_exp_f32_dev(float* x_dev, int64_t count, void* stream);
int sdcab_lambert_w_exp_f64_dev(double* x_dev, int64_t count, void* stream);

/* ------------------------------------------------------------- memory ---- */

/* Page-locked host memory for callers that want the host-buffer entry points
 * to overlap copies with kernels (any host memory is accepted). */
int sdcab_host_alloc(void** ptr, size_t bytes);
int sdcab_host_free(void* ptr);
/* Frees the device scratch the host-buffer entry points keep between calls. */
int sdcab_release_workspace(void);

#ifdef __cplusplus
}
#endif

#endif /* SDCA_B200_H */
