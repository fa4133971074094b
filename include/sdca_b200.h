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
  SDCAB_ERR_TOO_LARGE = -22,
  SDCAB_ERR_TIMEOUT = -23,       /* a bounded wait inside a kernel ran out */
  SDCAB_ERR_NCCL = -24           /* NCCL missing or a collective failed: sdcab_comm_last_error() */
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
  int32_t accurate_math;   /* 1: recompute t exactly from the final sets after variable
                            * fixing, as the reference does when it is compiled with
                            * SDCA_ACCURATE_MATH (include/sdca/prox/knapsack_eq.h:87-106);
                            * concerns knapsack_eq / _le / _le_biased and topk_simplex
                            * (+ biased), which end in that routine; 0 = the reference's
                            * default build */
} sdcab_prox_opts;

void sdcab_prox_opts_default(sdcab_prox_opts* opts);

/* Per-vector thresholds: prox(a) = max(lo, min(map(a - t), hi)); num_hi and
 * num_mid are the sizes of the sets the reference returns as iterator ranges
 * (include/sdca/prox/proxdef.h:29-67).  For the two-block operators every
 * vector has two consecutive records (first block, second block). */
typedef struct sdcab_thresholds {
  double t, lo, hi;
  int32_t num_hi, num_mid;
  int32_t status;    /* 0: solved.  bit 0: a bounded search ended without an admissible
                      * answer and the all-zero default stands in, which is what the
                      * reference returns silently (prox/topk_cone.h:131,
                      * knapsack_le_biased.h:85).  bit 1: a threshold is not finite
                      * (NaN or infinite entries in the vector; the reference asserts,
                      * proxdef.h:112) */
  int32_t reserved;
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

/* ---------------------------------------------------------------- eval ---- */

/* Objectives of matsdca_fit (src/matlab/mex_solve.cpp:643-715).  The ids name the
 * reference's objective classes (include/sdca/solver/objective/\*.h). */
enum {
  SDCAB_OBJ_L2_ENTROPY = 0,             /* softmax                                   */
  SDCAB_OBJ_L2_ENTROPY_TOPK = 1,        /* l2_entropy_topk                           */
  SDCAB_OBJ_L2_HINGE_TOPK = 2,          /* topk_hinge_alpha, gamma == 0              */
  SDCAB_OBJ_L2_HINGE_TOPK_SMOOTH = 3,   /* topk_hinge_alpha, gamma > 0               */
  SDCAB_OBJ_L2_TOPK_HINGE = 4,          /* topk_hinge_beta / msvm, gamma == 0        */
  SDCAB_OBJ_L2_TOPK_HINGE_SMOOTH = 5,   /* topk_hinge_beta / msvm_smooth, gamma > 0  */
  SDCAB_OBJ_L2_MULTILABEL_HINGE = 6,    /* mlsvm                                     */
  SDCAB_OBJ_L2_MULTILABEL_HINGE_SMOOTH = 7, /* mlsvm_smooth                          */
  SDCAB_OBJ_L2_MULTILABEL_ENTROPY = 8   /* mlsoftmax                                 */
};

typedef struct sdcab_objective {
  int32_t id;
  int32_t precision;  /* SDCAB_PRECISION_*: type of losses and accumulators */
  double c, gamma;
  int64_t k;
} sdcab_objective;

/* Maps an objective name and its parameters the way matsdca_fit does
 * (src/matlab/mex_solve.cpp:622-719): synonyms, gamma == 0 selecting the
 * non-smooth class, k == 1 for msvm / msvm_smooth / softmax, c > 0, gamma >= 0. */
int sdcab_objective_from_name(const char* name, double c, double gamma, int64_t k,
                              sdcab_objective* out);

enum { SDCAB_INPUT_FEATURES = 0, SDCAB_INPUT_KERNEL = 1 };

/* The evaluation record of the reference (include/sdca/solver/eval/types.h:12-172):
 * primal = primal_loss + primal_regularizer, dual = dual_loss - dual_regularizer;
 * rank_loss is used by the multilabel objectives, the accuracy histogram
 * (m entries, cumulative: entry j = top-(j+1) accuracy) by the multiclass ones. */
typedef struct sdcab_eval_record {
  double primal, dual, primal_loss, dual_loss, primal_regularizer, dual_regularizer;
  double rank_loss;
  double relative_gap;
} sdcab_eval_record;

/* Problem description shared by the evaluation and fit entry points.  Memory is
 * the reference's (include/sdca/solver/data/input.h): features are d x n
 * column major (example i at X + d*i), a kernel matrix is n_train x n column
 * major (column i at K + n_train*i), dual variables A are m x n_train column
 * major (example i at A + m*i), primal variables W are d x m column major.
 * Labels are 0-based; multilabel examples list their labels, sorted, at
 * labels[offsets[i] .. offsets[i+1]) (data/output.h:76-166). */
typedef struct sdcab_problem {
  int32_t input_kind;      /* SDCAB_INPUT_FEATURES or SDCAB_INPUT_KERNEL            */
  int32_t is_train;        /* 0: held-out set, only primal loss and accuracy        */
  int64_t d;               /* num_dimensions, or num_train_examples for a kernel    */
  int64_t n;               /* examples in this call (this rank's shard)             */
  int64_t m;               /* classes                                               */
  int64_t a_row_offset;    /* index of this shard's first example in A (train only) */
  const void* x;           /* features or kernel columns of the n examples          */
  const void* a;           /* dual variables (train sets, and kernel scores)        */
  const void* w;           /* primal variables (features)                           */
  const void* w0;          /* optional proximal centre W0 (features), or NULL       */
  const int64_t* labels;
  const int64_t* offsets;  /* multilabel only, n + 1 entries, offsets[0] == 0       */
  int32_t include_primal_regularizer; /* sharded runs: set on one rank only          */
  int32_t reserved;
} sdcab_problem;

/* Number of doubles in the sums vector of one evaluation: 8 scalars followed by
 * the m rank counts. */
#define SDCAB_EVAL_SUMS(m) (8 + (m))

/* Bytes of device scratch sdcab_eval_sums_*_dev needs (the score tile and the
 * per-block partial sums). */
size_t sdcab_eval_workspace_bytes(int64_t n, int64_t m, int64_t elem_size);

/*
 * Sums of one evaluation over the n examples described by `p` (all pointers in
 * p are device pointers): scores = W'x_i or A K_i for every example on the
 * device, then per-example loss, conjugate and rank.  Replaces the loop of
 * evaluate_dataset (include/sdca/solver/eval.h:15-51 with eval/scores.h,
 * eval/regularizer.h, eval/dual.h, eval/primal.h).  sums_dev receives
 * SDCAB_EVAL_SUMS(m) doubles:
 *   [0] sum of primal losses (before the objective's coefficient)
 *   [1] sum of dual losses   [2] primal regularizer   [3] dual regularizer
 *   [4] sum of rank losses   [5] number of examples
 *   [6] device error word (0 = none; sdcab_eval_finish then returns SDCAB_ERR_TIMEOUT)   [7] unused
 *   [8 + r] number of examples whose label is outranked by exactly r classes.
 * Rows are independent, so shards of examples are evaluated separately and
 * their sums added (one all-reduce over the ranks) before sdcab_eval_finish.
 * workspace_dev must hold sdcab_eval_workspace_bytes(...) bytes; NULL lets the
 * library use its own grow-only scratch (the first call then allocates).
 */
int sdcab_eval_sums_f32_dev(const sdcab_objective* obj, const sdcab_problem* p,
                            double* sums_dev, void* workspace_dev,
                            size_t workspace_bytes, void* stream);
int sdcab_eval_sums_f64_dev(const sdcab_objective* obj, const sdcab_problem* p,
                            double* sums_dev, void* workspace_dev,
                            size_t workspace_bytes, void* stream);

/*
 * sdcab_eval_sums_*_dev without any allocation (this entry point has no
 * counterpart in the reference).  Same arguments, same sums, but the scratch is
 * a fixed array of sdcab_eval_fixed_scratch_bytes() (16 MiB) that ships inside
 * the library and sits on every GPU that loads it until the process ends; no
 * cudaMalloc, cudaFree or other allocating call is made.  Meant for hosts that
 * must not allocate while they run -- a plug-in inside an application whose own
 * allocator already owns the device, or a loop that cannot take the device-wide
 * synchronisation of cudaMalloc.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and caches it; make that
 *     first call before any stream capture begins.
 *   - The number of classes is limited by the smaller of two bounds: 32 score
 *     rows, the rank histogram and the partial sums must fit the array (about
 *     130 000 float or 65 000 double classes), and four score rows must fit the
 *     shared memory of a thread block of the loss stage (about 14 000 float or
 *     7 000 double classes on a B200) -- the second one binds first.  Beyond
 *     either the call returns SDCAB_ERR_TOO_LARGE and
 *     sdcab_eval_fixed_scratch_error() holds the reason (it is cleared by a call
 *     that succeeds).  n is not limited: examples go through the array in chunks.
 *   - All calls on a device share the one array, which keeps what the last call
 *     left in it; the call clears what it accumulates into.  Two calls that
 *     overlap on the GPU (different streams, different host threads) race on
 *     it: run them one after the other.
 */
int sdcab_eval_sums_fixed_scratch_f32_dev(const sdcab_objective* obj, const sdcab_problem* p,
                                          double* sums_dev, void* stream);
int sdcab_eval_sums_fixed_scratch_f64_dev(const sdcab_objective* obj, const sdcab_problem* p,
                                          double* sums_dev, void* stream);
size_t sdcab_eval_fixed_scratch_bytes(void);
const char* sdcab_eval_fixed_scratch_error(void);

/*
 * The ranks of a sharded evaluation.  Examples are independent
 * (include/sdca/solver/eval.h:36-47), so each rank evaluates its shard into its own
 * sums vector and ONE all-reduce (sum, 8 + m doubles) gives every rank the sums of
 * the whole set; sdcab_eval_finish then runs on every rank.  The reference is a
 * single-process library and has no counterpart.  NCCL is bound at run time; a
 * NULL communicator stands for a single shard everywhere below.
 *   one process per GPU:  rank 0 calls sdcab_comm_unique_id and hands the
 *       SDCAB_COMM_ID_BYTES bytes to the other ranks by any means (a file, MPI, a
 *       socket); every rank then calls sdcab_comm_create with its device current;
 *   one process, several GPUs:  sdcab_comm_create_local fills `out[0 .. ngpus)`
 *       (devices = NULL means 0 .. ngpus - 1); collectives of the local ranks
 *       must then be issued from separate host threads or inside
 *       ncclGroupStart / ncclGroupEnd.
 * The primal regulariser is counted on the rank whose problem has
 * include_primal_regularizer set.
 */
typedef struct sdcab_comm sdcab_comm;
#define SDCAB_COMM_ID_BYTES 128
int sdcab_comm_unique_id(void* id_out);
int sdcab_comm_create(sdcab_comm** out, int nranks, int rank, const void* id);
int sdcab_comm_create_local(sdcab_comm** out, int ngpus, const int* devices);
int sdcab_comm_destroy(sdcab_comm* comm);
int sdcab_comm_rank(const sdcab_comm* comm);
int sdcab_comm_size(const sdcab_comm* comm);
const char* sdcab_comm_last_error(void);
/* In-place sums over the ranks on `stream` (asynchronous, like the kernels). */
int sdcab_comm_allreduce_f64(sdcab_comm* comm, double* buf_dev, int64_t count, void* stream);
int sdcab_comm_allreduce_f32(sdcab_comm* comm, float* buf_dev, int64_t count, void* stream);
/* sdcab_eval_sums_*_dev on this rank's shard followed by the all-reduce of the sums. */
int sdcab_eval_sums_sharded_f32_dev(const sdcab_objective* obj, const sdcab_problem* p,
                                    double* sums_dev, void* workspace_dev, size_t workspace_bytes,
                                    sdcab_comm* comm, void* stream);
int sdcab_eval_sums_sharded_f64_dev(const sdcab_objective* obj, const sdcab_problem* p,
                                    double* sums_dev, void* workspace_dev, size_t workspace_bytes,
                                    sdcab_comm* comm, void* stream);

/* Turns summed-up sums (host memory) into the record: applies the objective's
 * coefficient, forms primal / dual, normalises the accuracy histogram into
 * cumulative top-k accuracies (include/sdca/solver/eval/core.h:43-132,
 * objective/objective_base.h:108-128).  accuracy may be NULL. */
int sdcab_eval_finish(const sdcab_objective* obj, int64_t m, const double* sums,
                      sdcab_eval_record* record, double* accuracy);

/* Whole evaluation with host buffers on the current device (copies inside; the
 * examples are streamed through the device in chunks, uploads overlapping the
 * evaluation).  For a shard of a training set `a` points at the whole A and
 * a_row_offset names the shard's first example in it.  Labels and offsets are
 * checked as the reference checks them (include/sdca/solver/data/output.h:169-215:
 * range, offsets[0] == 0, between 1 and m - 1 labels per example, labels of an
 * example strictly increasing) and rejected with SDCAB_ERR_LABELS_RANGE; the
 * *_dev entry points trust the labels they are given.  Calls from several host
 * threads on one device are serialised. */
int sdcab_eval_f32(const sdcab_objective* obj, const sdcab_problem* host_problem,
                   sdcab_eval_record* record, double* accuracy);
int sdcab_eval_f64(const sdcab_objective* obj, const sdcab_problem* host_problem,
                   sdcab_eval_record* record, double* accuracy);

/* scores (n x m, example i at scores + m*i) = W'x_i or A K_i, device pointers:
 * the batched form of eval_scores (include/sdca/solver/eval/scores.h:9-47).
 * The float form synchronises the stream before it returns. */
int sdcab_scores_f32_dev(const sdcab_problem* p, float* scores_dev, void* stream);
int sdcab_scores_f64_dev(const sdcab_problem* p, double* scores_dev, void* stream);

/* ---------------------------------------------------------------- fit ---- */

/* solver_status of the reference (include/sdca/solver/solverdef.h:11-20). */
enum {
  SDCAB_FIT_NONE = 0,
  SDCAB_FIT_SOLVING = 1,
  SDCAB_FIT_SOLVED = 2,
  SDCAB_FIT_NO_PROGRESS = 3,
  SDCAB_FIT_MAX_EPOCH = 4,
  SDCAB_FIT_MAX_CPU_TIME = 5,
  SDCAB_FIT_MAX_WALL_TIME = 6,
  SDCAB_FIT_FAILED = 7
};

/* stopping_criteria of the reference (include/sdca/solver/solverdef.h:50-57). */
typedef struct sdcab_fit_criteria {
  double epsilon;         /* relative duality gap to reach                          */
  int64_t max_epoch;
  int64_t eval_epoch;     /* evaluate every eval_epoch epochs; 0: only at the end   */
  int32_t eval_on_start;
  int32_t recompute_primal; /* feature input: rebuild W = [W0 +] X A' before every
                             * evaluation, as the reference does when it is compiled with
                             * SDCA_ACCURATE_MATH (include/sdca/solver/eval/core.h:148-182);
                             * 0 = the reference's default build                       */
  double max_cpu_time;    /* seconds of processor time of the calling process (std::clock,
                           * like the reference's stopwatch); 0 = no limit            */
  double max_wall_time;   /* seconds of wall-clock time; 0 = no limit.  Both limits are
                           * checked where the reference checks them, after every epoch
                           * (include/sdca/solver/eval.h:95-107)                       */
} sdcab_fit_criteria;

typedef struct sdcab_fit_result {
  int32_t status;         /* SDCAB_FIT_*                                            */
  int32_t reserved;
  int64_t epoch;          /* epochs run                                             */
  int64_t num_evals;      /* records written to `evals`                             */
  double solve_seconds;   /* device time of the update steps                        */
  double eval_seconds;    /* device time of the evaluations                         */
  double cpu_seconds;     /* processor time of the calling process inside the fit   */
  double wall_seconds;    /* wall-clock time inside the fit                         */
} sdcab_fit_result;

/*
 * Primal variables from dual variables on the current device:
 * eval_recompute_primal of the reference (include/sdca/solver/eval/core.h:148-182,
 * sdca_blas_gemm(D, M, N, X, D, A, M, W, NoTrans, Trans[, 1, 1])), W = [W0 +] X A'.
 * x: d x n column major (features), a: m x n column major (dual variables),
 * w0: d x m column major or NULL, w: d x m column major (written).  All device
 * pointers; the sum over the examples runs in a fixed order.  Float data of 2048
 * examples and more runs on the tensor cores (3xTF32, float accuracy); that form
 * synchronises the stream before it returns and reports a wait that ran out inside
 * the kernel as SDCAB_ERR_TIMEOUT.
 */
int sdcab_primal_from_dual_f32_dev(const float* x, const float* a, const float* w0, float* w,
                                   int64_t d, int64_t m, int64_t n, void* stream);
int sdcab_primal_from_dual_f64_dev(const double* x, const double* a, const double* w0, double* w,
                                   int64_t d, int64_t m, int64_t n, void* stream);

/* The example order of the first num_epochs epochs of the reference's solver
 * for n training examples: a default-seeded std::minstd_rand driving
 * std::shuffle (as libstdc++ implements it) on one index vector that is kept
 * from epoch to epoch (include/sdca/solver.h:59,77-79,96-100).  perm (host)
 * receives num_epochs * n indices. */
int sdcab_epoch_permutations(int64_t n, int64_t num_epochs, int64_t* perm);

/*
 * SDCA fit on the current device: solver::solve of the reference
 * (include/sdca/solver.h:39-117) with update_variables
 * (include/sdca/solver/update.h:52-107) as the step and the evaluation above
 * after every eval_epoch epochs.  `train` holds device pointers: the kernel
 * matrix (n x n, input_kind SDCAB_INPUT_KERNEL, d == n) or the features
 * (d x n) in x, labels, and the variables the fit updates in place -- a
 * (m x n dual variables, read as the starting point) and, for features, w
 * (d x m primal variables, kept equal to X A').  Every objective of the list above
 * has its step (update_dual_variables of include/sdca/solver/objective/*.h);
 * multilabel objectives take labels / offsets as for the evaluation.  The top-k
 * hinge (beta) family, Crammer-Singer included, has a register-resident step for
 * up to 256 classes; the others run the general threshold routines.
 * The steps of one epoch are sequential by
 * definition; each step spreads its score product over the whole GPU.
 *   permutations: optional host array, max_epoch * n example indices (the
 *                 order of every epoch); NULL uses sdcab_epoch_permutations.
 *   evals:        host array of evals_cap records, one per evaluation in order
 *                 (later ones are dropped when it is full); may be NULL.
 * The call synchronises the stream at every evaluation.
 */
int sdcab_fit_f32_dev(const sdcab_objective* obj, const sdcab_problem* train,
                      const sdcab_fit_criteria* criteria, const int64_t* permutations,
                      sdcab_eval_record* evals, int64_t evals_cap,
                      sdcab_fit_result* result, void* stream);
int sdcab_fit_f64_dev(const sdcab_objective* obj, const sdcab_problem* train,
                      const sdcab_fit_criteria* criteria, const int64_t* permutations,
                      sdcab_eval_record* evals, int64_t evals_cap,
                      sdcab_fit_result* result, void* stream);

/* The same fit with host buffers on the current device: the problem is copied to
 * the device, a (and w for features) are read as the starting point and receive
 * the result -- what matsdca_fit does with its model struct
 * (src/matlab/mex_solve.cpp:780-800 and the make_context_* / solve_objective
 * helpers above it).  Labels and offsets are checked as in
 * include/sdca/solver/data/output.h:169-215 (SDCAB_ERR_LABELS_RANGE; labels are
 * 0-based here).  Synchronous. */
int sdcab_fit_f32(const sdcab_objective* obj, const sdcab_problem* host_train,
                  const sdcab_fit_criteria* criteria, const int64_t* permutations,
                  sdcab_eval_record* evals, int64_t evals_cap, sdcab_fit_result* result);
int sdcab_fit_f64(const sdcab_objective* obj, const sdcab_problem* host_train,
                  const sdcab_fit_criteria* criteria, const int64_t* permutations,
                  sdcab_eval_record* evals, int64_t evals_cap, sdcab_fit_result* result);

/*
 * The fit with its whole evaluation history and with held-out sets: after every
 * evaluation of the training set the reference evaluates each test set as well
 * (solver::evaluate_solution, include/sdca/solver.h:120-132; matsdca_fit takes the
 * sets as a cell array, src/matlab/mex_solve.cpp:473-501).  All arrays are host
 * memory owned by the caller; any of them may be NULL.
 */
typedef struct sdcab_fit_history {
  int64_t cap;                 /* evaluations the arrays below have room for               */
  int64_t num_tests;           /* held-out sets                                             */
  const sdcab_problem* tests;  /* num_tests problems with is_train = 0: x (features, or the
                                * kernel columns K_tst = X_trn' X_tst, d = n_train rows),
                                * n, labels, offsets; d and m as in the training set; a, w,
                                * w0 are taken from the training problem.  Same kind of
                                * pointers (device or host) as the training problem.        */
  sdcab_eval_record* train;    /* cap records of the training set                          */
  double* train_accuracy;      /* cap x m cumulative top-k accuracies (multiclass)         */
  int64_t* epoch;              /* cap: the epoch each evaluation was made after            */
  double* wall_seconds;        /* cap: wall-clock seconds since the start of the fit       */
  sdcab_eval_record* test;     /* cap x num_tests, evaluation e of set t at e*num_tests+t:
                                * primal_loss and rank_loss are set (eval_test,
                                * include/sdca/solver/eval/types.h:127-172)                 */
  double* test_accuracy;       /* cap x num_tests x m                                      */
} sdcab_fit_history;

int sdcab_fit_history_f32_dev(const sdcab_objective* obj, const sdcab_problem* train,
                              const sdcab_fit_criteria* criteria, const int64_t* permutations,
                              const sdcab_fit_history* history, sdcab_fit_result* result,
                              void* stream);
int sdcab_fit_history_f64_dev(const sdcab_objective* obj, const sdcab_problem* train,
                              const sdcab_fit_criteria* criteria, const int64_t* permutations,
                              const sdcab_fit_history* history, sdcab_fit_result* result,
                              void* stream);
/* Host buffers (training and test sets are copied to the device). */
int sdcab_fit_history_f32(const sdcab_objective* obj, const sdcab_problem* host_train,
                          const sdcab_fit_criteria* criteria, const int64_t* permutations,
                          const sdcab_fit_history* history, sdcab_fit_result* result);
int sdcab_fit_history_f64(const sdcab_objective* obj, const sdcab_problem* host_train,
                          const sdcab_fit_criteria* criteria, const int64_t* permutations,
                          const sdcab_fit_history* history, sdcab_fit_result* result);

/* ------------------------------------------------------------- front end ---- */

/*
 * matsdca_fit without Matlab (src/matlab/mex_solve.cpp:473-620, 722-800): options in,
 * model out, host buffers.  Defaults are the reference's: objective msvm_smooth
 * (mex_solve.cpp:15), c = 1, gamma = 1, k = 1, is_dual = 0, epsilon = 1e-3,
 * max_epoch = 1000, eval_epoch = 10, no time limits, double precision.
 */
typedef struct sdcab_dataset {
  int64_t n;               /* examples                                               */
  const void* x;           /* d x n features, or n_train x n Gram matrix columns     */
  const int64_t* labels;   /* 0-based or 1-based like the reference accepts them
                            * (data/output.h:169-182); multilabel: concatenated     */
  const int64_t* offsets;  /* multilabel objectives only: n + 1 offsets              */
} sdcab_dataset;

typedef struct sdcab_train_options {
  const char* objective;   /* a name sdcab_objective_from_name accepts; NULL = default */
  double c, gamma;
  int64_t k;
  int32_t is_dual;         /* 1: the data are Gram matrices (kernel input)          */
  int32_t precision;       /* SDCAB_PRECISION_*                                     */
  sdcab_fit_criteria criteria;
  int64_t num_dimensions;  /* d of the features; ignored for Gram matrices          */
  int64_t num_classes;     /* 0: largest label + 1, as the reference derives it     */
  const void* W0;          /* optional proximal centre, d x m (features only)       */
  int32_t warm_start;      /* 1: model.A (and model.W) hold the starting point;
                            * 0: they start from zero (W from W0 when W0 is given)  */
  int32_t reserved;
} sdcab_train_options;

void sdcab_train_options_default(sdcab_train_options* options);

/* The fields of matsdca_fit's model struct (mex_solve.cpp:153-376).  A and W are
 * caller-provided buffers (m x n and d x m; W may be NULL for Gram input); the
 * history arrays as in sdcab_fit_history (test sets come from the datasets). */
typedef struct sdcab_model {
  void* A;
  void* W;
  int64_t num_dimensions, num_examples, num_classes;
  int32_t is_dual, objective_id;
  char objective[40];
  double c, gamma;
  int64_t k;
  sdcab_fit_criteria criteria;
  int32_t status, data_precision, precision, labels_one_based;
  int64_t epoch;
  double cpu_time, wall_time, solve_time, eval_time, relative_gap;
  int64_t num_evals;
  sdcab_fit_history history;   /* cap and the arrays are set by the caller; tests is
                                * filled in by the call and not valid afterwards   */
} sdcab_model;

/* datasets[0] is the training set, the others are evaluated only. */
int sdcab_train_f32(const sdcab_dataset* datasets, int64_t num_datasets,
                    const sdcab_train_options* options, sdcab_model* model);
int sdcab_train_f64(const sdcab_dataset* datasets, int64_t num_datasets,
                    const sdcab_train_options* options, sdcab_model* model);

/* ------------------------------------------------------------- testing ---- */

/* Switches for the library's own tests; production code never needs them.
 *   "eval_chunk", n    examples per chunk of an evaluation (0 = automatic), so
 *                      that small problems run the chunk loop
 *   "gemm_simt", 0|1   1: score products on the CUDA cores even where the
 *                      tensor-core kernel applies
 *   "gemm_lose_a_tile", 0|1   1: the tensor-core product skips one operand tile
 *                      and runs with a short wait limit, so that one of its bounded
 *                      waits runs out and the call reports SDCAB_ERR_TIMEOUT
 *   "gemm_single_cta", 0|1   1: the one-CTA tensor-core kernel instead of the
 *                      paired-CTA one
 *   "gemm_write_hi", 0|1   1: the paired kernel stores the TF32 head of every
 *                      operand explicitly instead of leaving the truncation to the
 *                      tensor core
 *   "primal_simt", 0|1   1: sdcab_primal_from_dual_f32_dev on the CUDA cores
 *   "loss_general", 0|1   1: the general loss kernel (score rows in shared memory)
 *                      where the register-row kernel of the top-k hinge losses applies
 *   "gemm_f64_tile", 0..3   tile of the double-precision score products: 0 by
 *                      shape, 1 the 128-column block tile, 2 / 3 the pipelined
 *                      104-column tile with 64 / 128 rows per block
 * Returns SDCAB_ERR_ARG for an unknown name.  Not thread safe. */
int sdcab_test_set(const char* name, int64_t value);

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
