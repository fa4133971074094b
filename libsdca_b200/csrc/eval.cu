// Objective / duality-gap evaluation on the device.
//
//   scores   S (n x m, example-major) = X' W   (features: both operands have the
//            contraction index contiguous)  or  K' A' (kernel input), by a tiled
//            register-blocked GEMM written here;
//   losses   one warp per example: the score row is staged in shared memory and
//            the objective's loss, conjugate and rank come from the threshold
//            code of thresholds.cuh / losses.cuh; per-warp sums are combined per
//            block in a fixed order and the block partials by a single-block
//            kernel, so a run is reproducible bit for bit;
//   record   eval_finish on the host (eval_host.h).
//
// Examples are processed in chunks so that the score tile stays a few hundred
// megabytes whatever n is.  Replaces evaluate_dataset of the reference
// (include/sdca/solver/eval.h:15-51).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>
#include <vector>

#include "common_host.h"
#include "eval_host.h"
#include "gemm_blocked.cuh"
#include "gemm_pair.cuh"
#include "gemm_tc.cuh"
#include "losses.cuh"
#include "primal.h"

namespace sdcab {

static thread_local char g_fixed_scratch_error[160] = "";

// ---------------------------------------------------------------- losses ----
constexpr int kLossThreads = 128;
constexpr int kHistLocal = 256;  // ranks below this are counted per block first

struct LossArgs {
  ObjectiveParams obj;
  int m;
  long long n;             // examples in this chunk
  long long first;         // index of the chunk's first example within the call
  long long a_row_offset;  // index of the call's first example within A
  const long long* labels;
  const long long* offsets;
  int is_train, kernel_input;
  int m_pad, mask_words;
};

// block_partials[block][0..3] = primal loss, dual loss, dual regulariser term
// (0.5 <a_i, scores_i>, kernel input), rank loss; hist[r] += examples of rank r.
template <typename Data, typename R>
__global__ void __launch_bounds__(kLossThreads)
eval_loss_kernel(LossArgs g, const Data* __restrict__ scores, const Data* __restrict__ A,
                 double* __restrict__ block_partials, unsigned long long* __restrict__ hist) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ double warp_sums[kLossThreads / 32][4];
  __shared__ unsigned int local_hist[kHistLocal];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = kLossThreads / 32;
  Data* srow = reinterpret_cast<Data*>(smem_raw) + static_cast<size_t>(warp) * g.m_pad;
  unsigned* mask = reinterpret_cast<unsigned*>(reinterpret_cast<Data*>(smem_raw) +
                                               static_cast<size_t>(warps) * g.m_pad) +
                   static_cast<size_t>(warp) * g.mask_words;
  for (int i = threadIdx.x; i < kHistLocal; i += kLossThreads) local_hist[i] = 0;
  __syncthreads();
  const bool ml = objective_is_multilabel(g.obj.id);
  const int m = g.m;
  double primal = 0, dual = 0, reg = 0, rank_loss = 0;
  for (long long e = static_cast<long long>(blockIdx.x) * warps + warp; e < g.n;
       e += static_cast<long long>(gridDim.x) * warps) {
    const Data* s_g = scores + e * m;
    for (int i = lane; i < m; i += 32) srow[i] = s_g[i];
    const long long ex = g.first + e;  // example index within the call
    const Data* a = (g.is_train && A) ? A + (g.a_row_offset + ex) * m : nullptr;
    __syncwarp();
    if (!ml) {
      const int y = static_cast<int>(g.labels[ex]);
      int rank;
      primal += static_cast<double>(multiclass_primal_loss<R, Data>(g.obj, srow, m, y, rank));
      if (lane == 0) {
        if (rank < kHistLocal) atomicAdd(&local_hist[rank], 1u);
        else atomicAdd(&hist[rank], 1ull);
      }
      if (a) dual += static_cast<double>(multiclass_dual_loss<R, Data>(g.obj, a, m, y));
    } else {
      const long long off = g.offsets[ex];
      const int nl = static_cast<int>(g.offsets[ex + 1] - off);
      for (int w = lane; w < g.mask_words; w += 32) mask[w] = 0u;
      __syncwarp();
      for (int q = lane; q < nl; q += 32) {
        const int c = static_cast<int>(g.labels[off + q]);
        atomicOr(&mask[c >> 5], 1u << (c & 31));
      }
      __syncwarp();
      R rl;
      primal += static_cast<double>(
          multilabel_primal_loss<R, Data>(g.obj, srow, m, mask, g.labels + off, nl, rl));
      rank_loss += static_cast<double>(rl);
      if (a) dual += static_cast<double>(multilabel_dual_loss<R, Data>(g.obj, a, m, mask, nl));
    }
    if (a && g.kernel_input) {
      // 0.5 <a_i, scores_i>: eval/regularizer.h:82-98, objective_base.h:92-105
      R dot = 0;
      for (int i = lane; i < m; i += 32) dot += static_cast<R>(a[i]) * static_cast<R>(srow[i]);
      reg += static_cast<double>(warp_sum(dot)) * 0.5;
    }
    __syncwarp();
  }
  if (lane == 0) {
    warp_sums[warp][0] = primal; warp_sums[warp][1] = dual;
    warp_sums[warp][2] = reg; warp_sums[warp][3] = rank_loss;
  }
  __syncthreads();
  if (threadIdx.x < 4) {
    double s = 0;
    for (int w = 0; w < warps; ++w) s += warp_sums[w][threadIdx.x];
    block_partials[static_cast<size_t>(blockIdx.x) * 4 + threadIdx.x] = s;
  }
  for (int i = threadIdx.x; i < kHistLocal && i < m; i += kLossThreads)
    if (local_hist[i]) atomicAdd(&hist[i], static_cast<unsigned long long>(local_hist[i]));
}

}  // namespace sdcab
#include "loss_rows.cuh"
namespace sdcab {

// sums[0..4] += block partials.  One block of 256 threads: thread t adds the
// partials of blocks t, t + 256, ... in order, then a fixed tree combines the
// 256 values, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256)
combine_partials_kernel(const double* __restrict__ partials, int blocks,
                        double* __restrict__ sums) {
  __shared__ double sh[4][256];
  const int t = threadIdx.x;
  double s[4] = {0, 0, 0, 0};
  for (int b = t; b < blocks; b += 256) {
#pragma unroll
    for (int q = 0; q < 4; ++q) s[q] += partials[static_cast<size_t>(b) * 4 + q];
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) sh[q][t] = s[q];
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (t < o) {
#pragma unroll
      for (int q = 0; q < 4; ++q) sh[q][t] += sh[q][t + o];
    }
    __syncthreads();
  }
  if (t == 0) {
    // [0] primal loss, [1] dual loss, [2]+[3] regularisers, [4] rank loss
    sums[0] += sh[0][0];
    sums[1] += sh[1][0];
    sums[2] += sh[2][0]; sums[3] += sh[2][0];
    sums[4] += sh[3][0];
  }
}

__global__ void hist_to_sums_kernel(const unsigned long long* __restrict__ hist, int m,
                                    double* __restrict__ sums) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m; i += gridDim.x * blockDim.x)
    sums[8 + i] = static_cast<double>(hist[i]);
}

// 0.5 <W, W> and <W0, W> with double accumulation: two-stage, fixed order.
template <typename Data>
__global__ void __launch_bounds__(256)
dot_partials_kernel(const Data* __restrict__ w, const Data* __restrict__ w0, long long count,
                    double* __restrict__ partials) {
  __shared__ double sh[2][256];
  double ww = 0, w0w = 0;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const double v = static_cast<double>(w[i]);
    ww += v * v;
    if (w0) w0w += static_cast<double>(w0[i]) * v;
  }
  sh[0][threadIdx.x] = ww; sh[1][threadIdx.x] = w0w;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      sh[0][threadIdx.x] += sh[0][threadIdx.x + o];
      sh[1][threadIdx.x] += sh[1][threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    partials[2 * blockIdx.x] = sh[0][0];
    partials[2 * blockIdx.x + 1] = sh[1][0];
  }
}

// eval/regularizer.h:22-63 with objective_base.h:59-89
__global__ void __launch_bounds__(256)
regularizer_combine_kernel(const double* __restrict__ partials, int blocks, int has_w0,
                           double* __restrict__ sums) {
  __shared__ double sh[2][256];
  const int t = threadIdx.x;
  double ww = 0, w0w = 0;
  for (int b = t; b < blocks; b += 256) { ww += partials[2 * b]; w0w += partials[2 * b + 1]; }
  sh[0][t] = ww; sh[1][t] = w0w;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (t < o) { sh[0][t] += sh[0][t + o]; sh[1][t] += sh[1][t + o]; }
    __syncthreads();
  }
  if (t == 0) {
    const double regul = sh[0][0] / 2;
    sums[2] += has_w0 ? regul - sh[1][0] : regul;
    sums[3] += regul;
  }
}

// sums[6] carries the error word of the tensor-core GEMM (0 = none): a bounded
// wait inside that kernel ran out; sdcab_eval_finish turns it into a status.
__global__ void report_gemm_error_kernel(const int* err, double* sums) {
  if (threadIdx.x == 0) sums[6] = static_cast<double>(*err);
}

__global__ void set_count_kernel(double* sums, double n) {
  if (threadIdx.x == 0) sums[5] = n;
}

// ----------------------------------------------------------------- layout ----
struct EvalLayout {
  long long chunk;       // examples per chunk
  size_t scores_bytes;   // chunk * m * elem, rounded up
  int max_blocks;
  size_t partials_bytes, hist_bytes, total;
  size_t err_offset;     // one int: error word of the tensor-core GEMM
};

// Settings that only tests change (sdcab_test_set): a forced chunk length so that
// small problems exercise the chunk loop, and the CUDA-core product in place of the
// tensor-core one.  0 / 0 is the library's normal behaviour.
static long long g_test_eval_chunk = 0;
static int g_test_force_simt = 0;
static int g_test_lose_a_tile = 0;
static int g_test_single_cta = 0;   // the one-CTA tensor-core kernel instead of the paired one
static int g_test_write_hi = 0;     // the paired kernel writes the TF32 head explicitly
static int g_test_loss_general = 0; // the general loss kernel where the register-row one applies

// Chunks are bounded so that the product's grid (one row of thread blocks per 128
// examples in grid.y for the CUDA-core kernel) stays inside the launch limits.
constexpr long long kMaxChunkRows = 65535LL * 64;

static EvalLayout eval_layout(long long n, long long m, long long elem, int sm_count) {
  EvalLayout L;
  const long long budget = 256LL << 20;
  long long chunk = std::max<long long>(128, budget / std::max<long long>(1, m * elem));
  if (g_test_eval_chunk > 0) chunk = g_test_eval_chunk;
  chunk = std::min(chunk, kMaxChunkRows);
  chunk = std::min(chunk, std::max<long long>(n, 1));
  L.chunk = chunk;
  L.scores_bytes = (static_cast<size_t>(chunk) * m * elem + 255) & ~static_cast<size_t>(255);
  L.max_blocks = std::max(1, sm_count) * 16;
  L.partials_bytes = (static_cast<size_t>(L.max_blocks) * 4 * sizeof(double) + 255) & ~static_cast<size_t>(255);
  L.hist_bytes = (static_cast<size_t>(m) * sizeof(unsigned long long) + 255) & ~static_cast<size_t>(255);
  L.err_offset = L.scores_bytes + L.partials_bytes + L.hist_bytes;
  L.total = L.err_offset + 256;
  return L;
}

static int check_problem(const sdcab_objective* obj, const sdcab_problem* p) {
  if (!obj || !p) return SDCAB_ERR_ARG;
  if (p->n <= 0 || p->m <= 0 || p->d <= 0) return SDCAB_ERR_NOT_EMPTY;
  if (p->m > 0x7fffffffLL || p->d > 0x7fffffffLL) return SDCAB_ERR_TOO_LARGE;
  if (p->m < 2) return SDCAB_ERR_NUM_DIM;
  int rc = check_objective(obj, p->m);
  if (rc) return rc;
  if (!p->x || !p->labels) return SDCAB_ERR_ARG;
  if (p->input_kind == SDCAB_INPUT_FEATURES) {
    if (!p->w) return SDCAB_ERR_ARG;
  } else if (p->input_kind == SDCAB_INPUT_KERNEL) {
    if (!p->a) return SDCAB_ERR_ARG;
  } else {
    return SDCAB_ERR_ARG;
  }
  if (p->is_train && !p->a) return SDCAB_ERR_ARG;
  if (objective_is_multilabel(obj->id) && !p->offsets) return SDCAB_ERR_ARG;
  return SDCAB_OK;
}

// scores of examples [first, first + count) into `out` (count x m)
// The float feature GEMM runs on the tensor cores (gemm_tc.cuh) when the caller
// provides an error word and the operands meet TMA's alignment rules.
inline bool tensor_core_gemm_enabled() { return g_test_force_simt == 0; }

inline int scores_tc(const float* X, const float* W, float* out, int M, int N, int K, long long ld,
                     int* tc_err, cudaStream_t stream) {
  if (!g_test_single_cta) {
    const int rc = tc2::launch(X, W, out, M, N, K, ld, ld, N, tc_err, g_test_write_hi != 0,
                               g_test_lose_a_tile != 0, stream);
    // NOT_IMPLEMENTED: the build's register count does not fit the paired kernel's
    // hand-over of registers; the one-CTA kernel takes the product instead
    if (rc != SDCAB_ERR_NOT_IMPLEMENTED) return rc;
  }
  return tc::launch(X, W, out, M, N, K, ld, ld, N, tc_err, stream);
}
inline int scores_tc(const double*, const double*, double*, int, int, int, long long, int*,
                     cudaStream_t) {
  return SDCAB_ERR_NOT_IMPLEMENTED;
}
inline bool scores_tc_usable(const float* X, const float* W, long long ld) { return tc::usable(X, W, ld, ld); }
inline bool scores_tc_usable(const double*, const double*, long long) { return false; }

template <typename Data>
int scores_chunk(const sdcab_problem* p, long long first, long long count, Data* out,
                 cudaStream_t stream, int* tc_err = nullptr) {
  const Data* X = static_cast<const Data*>(p->x) + first * p->d;
  const int M = static_cast<int>(count), N = static_cast<int>(p->m), K = static_cast<int>(p->d);
  if (p->input_kind == SDCAB_INPUT_FEATURES) {
    // S[i][j] = sum_l X[i][l] W[j][l]   (eval/scores.h:9-26)
    if (tc_err && tensor_core_gemm_enabled() && K >= 32 &&
        scores_tc_usable(X, static_cast<const Data*>(p->w), p->d))
      return scores_tc(X, static_cast<const Data*>(p->w), out, M, N, K, p->d, tc_err, stream);
    return launch_gemm<Data>(X, static_cast<const Data*>(p->w), out, M, N, K, p->d, p->d, p->m,
                             true, stream);
  }
  // S[i][j] = sum_l K[i][l] A[l][j]     (eval/scores.h:30-47)
  return launch_gemm<Data>(X, static_cast<const Data*>(p->a), out, M, N, K, p->d, p->m, p->m,
                           false, stream);
}

template <typename Data>
int eval_sums_dev(const sdcab_objective* obj, const sdcab_problem* p, double* sums,
                  void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  int rc = check_problem(obj, p);
  if (rc) return rc;
  if (!sums) return SDCAB_ERR_ARG;
  DeviceInfo info;
  rc = get_device_info(&info);
  if (rc) return rc;
  const long long m = p->m, n = p->n;
  const EvalLayout L = eval_layout(n, m, sizeof(Data), info.sm_count);
  if (!workspace) {
    rc = workspace_reserve(2, L.total, &workspace);
    if (rc) return rc;
  } else if (workspace_bytes < L.total) {
    return SDCAB_ERR_ARG_RANGE;
  }
  unsigned char* base = static_cast<unsigned char*>(workspace);
  Data* scores = reinterpret_cast<Data*>(base);
  double* partials = reinterpret_cast<double*>(base + L.scores_bytes);
  unsigned long long* hist = reinterpret_cast<unsigned long long*>(base + L.scores_bytes + L.partials_bytes);

  int* tc_err = reinterpret_cast<int*>(base + L.err_offset);
  SDCAB_CUDA_TRY(cudaMemsetAsync(sums, 0, sizeof(double) * SDCAB_EVAL_SUMS(m), stream));
  SDCAB_CUDA_TRY(cudaMemsetAsync(hist, 0, sizeof(unsigned long long) * m, stream));
  SDCAB_CUDA_TRY(cudaMemsetAsync(tc_err, 0, sizeof(int), stream));
  set_count_kernel<<<1, 32, 0, stream>>>(sums, static_cast<double>(n));

  if (p->is_train && p->input_kind == SDCAB_INPUT_FEATURES && p->include_primal_regularizer) {
    const long long count = p->d * m;
    const int blocks = static_cast<int>(std::min<long long>(L.max_blocks / 2, (count + 255) / 256));
    dot_partials_kernel<Data><<<blocks, 256, 0, stream>>>(
        static_cast<const Data*>(p->w), static_cast<const Data*>(p->w0), count, partials);
    regularizer_combine_kernel<<<1, 256, 0, stream>>>(partials, blocks, p->w0 ? 1 : 0, sums);
  }

  LossArgs g;
  g.obj = to_params(obj);
  g.m = static_cast<int>(m);
  g.a_row_offset = p->a_row_offset;
  g.labels = reinterpret_cast<const long long*>(p->labels);
  g.offsets = reinterpret_cast<const long long*>(p->offsets);
  g.is_train = p->is_train;
  g.kernel_input = (p->input_kind == SDCAB_INPUT_KERNEL);
  g.m_pad = static_cast<int>((m + 15) & ~15LL);
  g.mask_words = static_cast<int>((m + 31) / 32);
  const int warps = kLossThreads / 32;
  const size_t smem = static_cast<size_t>(warps) * g.m_pad * sizeof(Data) +
                      static_cast<size_t>(warps) * g.mask_words * sizeof(unsigned);
  if (smem > info.smem_optin) return SDCAB_ERR_TOO_LARGE;
  const bool fl = (obj->precision == SDCAB_PRECISION_FLOAT);
  auto kd = eval_loss_kernel<Data, double>;
  auto kf = eval_loss_kernel<Data, float>;
  if (smem > 48 * 1024) {
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kd, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  }
  for (long long first = 0; first < n; first += L.chunk) {
    const long long count = std::min(L.chunk, n - first);
    rc = scores_chunk<Data>(p, first, count, scores, stream, tc_err);
    if (rc) return rc;
    g.n = count; g.first = first;
    const int blocks = static_cast<int>(std::max<long long>(
        1, std::min<long long>(L.max_blocks, (count + warps - 1) / warps)));
    const Data* A = static_cast<const Data*>(p->a);
    bool launched = false;
    if constexpr (std::is_same<Data, float>::value) {
      if (!g_test_loss_general && loss_rows_usable(g, scores, A)) {
        rc = fl ? launch_loss_rows<float>(g, scores, A, partials, hist, blocks, info.smem_optin, stream)
                : launch_loss_rows<double>(g, scores, A, partials, hist, blocks, info.smem_optin, stream);
        if (rc) return rc;
        launched = true;
      }
    }
    if (!launched) {
      if (fl) kf<<<blocks, kLossThreads, smem, stream>>>(g, scores, A, partials, hist);
      else kd<<<blocks, kLossThreads, smem, stream>>>(g, scores, A, partials, hist);
    }
    combine_partials_kernel<<<1, 256, 0, stream>>>(partials, blocks, sums);
  }
  hist_to_sums_kernel<<<std::max(1, static_cast<int>((m + 255) / 256)), 256, 0, stream>>>(
      hist, static_cast<int>(m), sums);
  report_gemm_error_kernel<<<1, 32, 0, stream>>>(tc_err, sums);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

// Host buffers.  W (or A for a kernel input), the labels and W0 stay on the device
// for the whole call; the examples -- and, for a training set given by features,
// the rows of A that belong to them -- go through three device buffers on three
// streams, so that the upload of one chunk overlaps the evaluation of the chunk
// before it.  Each chunk's sums land in page-locked host memory and are added up
// in chunk order once the last stream has drained.  Device scratch comes from
// the library's grow-only workspace, so only the first call of a size allocates.
template <typename Data>
int eval_host(const sdcab_objective* obj, const sdcab_problem* hp, sdcab_eval_record* rec,
              double* accuracy) {
  int rc = check_problem(obj, hp);
  if (rc) return rc;
  if (!rec) return SDCAB_ERR_ARG;
  const long long m = hp->m, n = hp->n, d = hp->d;
  const bool kernel = (hp->input_kind == SDCAB_INPUT_KERNEL);
  const bool ml = objective_is_multilabel(obj->id);
  // include/sdca/solver/data/output.h:169-215: bad labels are an argument error,
  // they never reach a kernel
  rc = validate_labels(hp->labels, hp->offsets, n, m, ml);
  if (rc) return rc;
  if (hp->a_row_offset < 0) return SDCAB_ERR_ARG_RANGE;
  if (kernel && hp->is_train && hp->a_row_offset + n > d) return SDCAB_ERR_ARG_RANGE;
  DeviceInfo info;
  rc = get_device_info(&info);
  if (rc) return rc;
  std::lock_guard<std::mutex> call_lock(*host_call_mutex());

  const size_t elem = sizeof(Data);
  const bool a_chunked = hp->is_train && !kernel;  // A rows travel with their examples
  long long chunk = std::max<long long>(1, (64LL << 20) / std::max<long long>(1, d * static_cast<long long>(elem)));
  if (g_test_eval_chunk > 0) chunk = g_test_eval_chunk;
  chunk = std::min(chunk, n);
  const long long num_chunks = (n + chunk - 1) / chunk;
  const long long num_labels = ml ? hp->offsets[n] : n;
  const size_t sums_count = SDCAB_EVAL_SUMS(m);
  constexpr int kBuf = 3;
  auto round256 = [](size_t b) { return (b + 255) & ~static_cast<size_t>(255); };
  const EvalLayout L = eval_layout(chunk, m, static_cast<long long>(elem), info.sm_count);
  const size_t x_bytes = round256(static_cast<size_t>(chunk) * d * elem);
  const size_t a_chunk_bytes = a_chunked ? round256(static_cast<size_t>(chunk) * m * elem) : 0;
  const size_t sums_bytes = round256(sums_count * sizeof(double));
  const size_t slot_bytes = x_bytes + a_chunk_bytes + round256(L.total) + sums_bytes;
  const size_t a_full_bytes = (kernel && hp->a) ? round256(static_cast<size_t>(d) * m * elem) : 0;
  const size_t w_bytes = hp->w ? round256(static_cast<size_t>(d) * m * elem) : 0;
  const size_t w0_bytes = hp->w0 ? w_bytes : 0;
  const size_t lab_bytes = round256(static_cast<size_t>(num_labels) * sizeof(int64_t));
  const size_t off_bytes = ml ? round256(static_cast<size_t>(n + 1) * sizeof(int64_t)) : 0;
  void* arena = nullptr;
  rc = workspace_reserve(4, kBuf * slot_bytes + a_full_bytes + w_bytes + w0_bytes + lab_bytes + off_bytes,
                         &arena);
  if (rc) return rc;
  void* pinned = nullptr;
  rc = pinned_reserve(static_cast<size_t>(num_chunks) * sums_bytes, &pinned);
  if (rc) return rc;
  cudaStream_t streams[kBuf];
  rc = pipeline_streams(kBuf, streams);
  if (rc) return rc;

  unsigned char* base = static_cast<unsigned char*>(arena);
  unsigned char* slots = base;
  unsigned char* cur = base + kBuf * slot_bytes;
  void* dA = nullptr; void* dW = nullptr; void* dW0 = nullptr;
  if (a_full_bytes) { dA = cur; cur += a_full_bytes; }
  if (w_bytes) { dW = cur; cur += w_bytes; }
  if (w0_bytes) { dW0 = cur; cur += w0_bytes; }
  int64_t* dLab = reinterpret_cast<int64_t*>(cur); cur += lab_bytes;
  int64_t* dOff = ml ? reinterpret_cast<int64_t*>(cur) : nullptr;

  // resident operands on the first stream; the other streams wait for them
  cudaStream_t s0 = streams[0];
  if (dA) SDCAB_CUDA_TRY(cudaMemcpyAsync(dA, hp->a, static_cast<size_t>(d) * m * elem, cudaMemcpyHostToDevice, s0));
  if (dW) SDCAB_CUDA_TRY(cudaMemcpyAsync(dW, hp->w, static_cast<size_t>(d) * m * elem, cudaMemcpyHostToDevice, s0));
  if (dW0) SDCAB_CUDA_TRY(cudaMemcpyAsync(dW0, hp->w0, static_cast<size_t>(d) * m * elem, cudaMemcpyHostToDevice, s0));
  SDCAB_CUDA_TRY(cudaMemcpyAsync(dLab, hp->labels, static_cast<size_t>(num_labels) * sizeof(int64_t),
                                 cudaMemcpyHostToDevice, s0));
  if (ml) SDCAB_CUDA_TRY(cudaMemcpyAsync(dOff, hp->offsets, static_cast<size_t>(n + 1) * sizeof(int64_t),
                                         cudaMemcpyHostToDevice, s0));
  SDCAB_CUDA_TRY(cudaStreamSynchronize(s0));

  long long index = 0;
  for (long long first = 0; first < n; first += chunk, ++index) {
    const long long count = std::min(chunk, n - first);
    const int slot = static_cast<int>(index % kBuf);
    cudaStream_t s = streams[slot];
    // a slot is reused only after the stream that owns it has drained
    if (index >= kBuf) SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
    unsigned char* sb = slots + static_cast<size_t>(slot) * slot_bytes;
    Data* dX = reinterpret_cast<Data*>(sb);
    Data* dAc = a_chunked ? reinterpret_cast<Data*>(sb + x_bytes) : nullptr;
    void* ws = sb + x_bytes + a_chunk_bytes;
    double* dSums = reinterpret_cast<double*>(sb + x_bytes + a_chunk_bytes + round256(L.total));
    SDCAB_CUDA_TRY(cudaMemcpyAsync(dX, static_cast<const Data*>(hp->x) + first * d,
                                   static_cast<size_t>(count) * d * elem, cudaMemcpyHostToDevice, s));
    sdcab_problem dp = *hp;
    dp.x = dX; dp.w = dW; dp.w0 = dW0;
    dp.n = count;
    if (a_chunked) {
      // the chunk's own rows of A: row 0 of the buffer is example `first` of the shard
      SDCAB_CUDA_TRY(cudaMemcpyAsync(dAc, static_cast<const Data*>(hp->a) + (hp->a_row_offset + first) * m,
                                     static_cast<size_t>(count) * m * elem, cudaMemcpyHostToDevice, s));
      dp.a = dAc; dp.a_row_offset = 0;
    } else {
      dp.a = dA; dp.a_row_offset = hp->a_row_offset + first;
    }
    dp.labels = ml ? dLab : dLab + first;
    dp.offsets = ml ? dOff + first : nullptr;
    dp.include_primal_regularizer = (first == 0) ? hp->include_primal_regularizer : 0;
    rc = eval_sums_dev<Data>(obj, &dp, dSums, ws, L.total, s);
    if (rc) return rc;
    SDCAB_CUDA_TRY(cudaMemcpyAsync(static_cast<unsigned char*>(pinned) + static_cast<size_t>(index) * sums_bytes,
                                   dSums, sums_count * sizeof(double), cudaMemcpyDeviceToHost, s));
  }
  for (int i = 0; i < kBuf; ++i) SDCAB_CUDA_TRY(cudaStreamSynchronize(streams[i]));
  std::vector<double> total(sums_count, 0.0);
  for (long long c = 0; c < num_chunks; ++c) {
    const double* part = reinterpret_cast<const double*>(static_cast<unsigned char*>(pinned) +
                                                         static_cast<size_t>(c) * sums_bytes);
    for (size_t i = 0; i < sums_count; ++i) total[i] += part[i];
  }
  return eval_finish(obj, m, total.data(), rec, accuracy);
}

// ------------------------------------------------- fixed-scratch variant ----
// The evaluation above needs device scratch (the score tile, the per-block
// partial sums and the rank histogram).  This variant keeps that scratch in a
// fixed array that is part of the library image, so it never asks the CUDA
// runtime (or anybody else) for memory.  It serves hosts that may not allocate
// while they run: a plug-in living inside an application whose own allocator
// has already claimed the device and treats every foreign cudaMalloc as a
// failure or a fragmentation hazard, and control loops that cannot afford the
// device-wide synchronisation a cudaMalloc / cudaFree implies.
//
// The array exists once per GPU that loads the library and stays resident until
// the process exits.  In host code its name is only a handle: the device address
// is looked up with cudaGetSymbolAddress the first time the entry point runs on
// a device (with that device current) and cached.
constexpr size_t kFixedScratchBytes = static_cast<size_t>(16) << 20;
static __device__ __align__(256) unsigned char g_fixed_scratch[kFixedScratchBytes];

static void* g_fixed_scratch_ptr[64] = {nullptr};
static std::mutex g_fixed_scratch_mutex;

static int fixed_scratch_address(void** out) {
  int dev = -1;
  SDCAB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return SDCAB_ERR_NO_DEVICE;
  std::lock_guard<std::mutex> lock(g_fixed_scratch_mutex);
  if (!g_fixed_scratch_ptr[dev]) {
    void* ptr = nullptr;
    SDCAB_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_fixed_scratch));
    g_fixed_scratch_ptr[dev] = ptr;
  }
  *out = g_fixed_scratch_ptr[dev];
  return SDCAB_OK;
}

// Same sequence of kernels as eval_sums_dev, with the chunk length derived from
// the fixed scratch instead of from a budget.
template <typename Data>
int eval_sums_fixed_scratch(const sdcab_objective* obj, const sdcab_problem* p, double* sums,
                            cudaStream_t stream) {
  int rc = check_problem(obj, p);
  if (rc) return rc;
  if (!sums) return SDCAB_ERR_ARG;
  DeviceInfo info;
  rc = get_device_info(&info);
  if (rc) return rc;
  void* scratch = nullptr;
  rc = fixed_scratch_address(&scratch);
  if (rc) return rc;
  const long long m = p->m, n = p->n;
  const int max_blocks = std::max(1, info.sm_count) * 16;
  const size_t partials_bytes = (static_cast<size_t>(max_blocks) * 4 * sizeof(double) + 255) & ~static_cast<size_t>(255);
  const size_t hist_bytes = (static_cast<size_t>(m) * sizeof(unsigned long long) + 255) & ~static_cast<size_t>(255);
  const size_t row_bytes = static_cast<size_t>(m) * sizeof(Data);
  g_fixed_scratch_error[0] = 0;
  // at least 32 score rows must fit beside the partial sums, the histogram and the
  // error word of the tensor-core product
  constexpr size_t kErrBytes = 256;
  if (partials_bytes + hist_bytes + kErrBytes + 32 * row_bytes + 256 > kFixedScratchBytes) {
    std::snprintf(g_fixed_scratch_error, sizeof(g_fixed_scratch_error),
                  "the fixed scratch of %zu bytes cannot hold 32 score rows of %lld classes",
                  kFixedScratchBytes, m);
    return SDCAB_ERR_TOO_LARGE;
  }
  const size_t scores_room =
      (kFixedScratchBytes - partials_bytes - hist_bytes - kErrBytes) & ~static_cast<size_t>(255);
  const long long chunk = std::min<long long>(
      std::min<long long>(n, kMaxChunkRows), static_cast<long long>(scores_room / row_bytes));
  unsigned char* base = static_cast<unsigned char*>(scratch);
  Data* scores = reinterpret_cast<Data*>(base);
  double* partials = reinterpret_cast<double*>(base + scores_room);
  unsigned long long* hist = reinterpret_cast<unsigned long long*>(base + scores_room + partials_bytes);
  int* tc_err = reinterpret_cast<int*>(base + scores_room + partials_bytes + hist_bytes);

  // the array keeps whatever the previous call left: everything that is
  // accumulated into starts from zero here, the rest is overwritten before use
  SDCAB_CUDA_TRY(cudaMemsetAsync(sums, 0, sizeof(double) * SDCAB_EVAL_SUMS(m), stream));
  SDCAB_CUDA_TRY(cudaMemsetAsync(hist, 0, sizeof(unsigned long long) * m, stream));
  SDCAB_CUDA_TRY(cudaMemsetAsync(tc_err, 0, sizeof(int), stream));
  set_count_kernel<<<1, 32, 0, stream>>>(sums, static_cast<double>(n));
  if (p->is_train && p->input_kind == SDCAB_INPUT_FEATURES && p->include_primal_regularizer) {
    const long long count = p->d * m;
    const int blocks = static_cast<int>(std::min<long long>(max_blocks / 2, (count + 255) / 256));
    dot_partials_kernel<Data><<<blocks, 256, 0, stream>>>(
        static_cast<const Data*>(p->w), static_cast<const Data*>(p->w0), count, partials);
    regularizer_combine_kernel<<<1, 256, 0, stream>>>(partials, blocks, p->w0 ? 1 : 0, sums);
  }
  LossArgs g;
  g.obj = to_params(obj);
  g.m = static_cast<int>(m);
  g.a_row_offset = p->a_row_offset;
  g.labels = reinterpret_cast<const long long*>(p->labels);
  g.offsets = reinterpret_cast<const long long*>(p->offsets);
  g.is_train = p->is_train;
  g.kernel_input = (p->input_kind == SDCAB_INPUT_KERNEL);
  g.m_pad = static_cast<int>((m + 15) & ~15LL);
  g.mask_words = static_cast<int>((m + 31) / 32);
  const int warps = kLossThreads / 32;
  const size_t smem = static_cast<size_t>(warps) * g.m_pad * sizeof(Data) +
                      static_cast<size_t>(warps) * g.mask_words * sizeof(unsigned);
  if (smem > info.smem_optin) {
    // the loss stage stages four score rows per thread block in shared memory: this
    // bound (about 14 000 float or 7 000 double classes) is the one that binds first
    std::snprintf(g_fixed_scratch_error, sizeof(g_fixed_scratch_error),
                  "%lld classes need %zu bytes of shared memory per thread block, the device offers %zu",
                  m, smem, info.smem_optin);
    return SDCAB_ERR_TOO_LARGE;
  }
  const bool fl = (obj->precision == SDCAB_PRECISION_FLOAT);
  auto kd = eval_loss_kernel<Data, double>;
  auto kf = eval_loss_kernel<Data, float>;
  if (smem > 48 * 1024) {
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kd, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kf, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  }
  for (long long first = 0; first < n; first += chunk) {
    const long long count = std::min(chunk, n - first);
    rc = scores_chunk<Data>(p, first, count, scores, stream, tc_err);
    if (rc) return rc;
    g.n = count; g.first = first;
    const int blocks = static_cast<int>(std::max<long long>(
        1, std::min<long long>(max_blocks, (count + warps - 1) / warps)));
    const Data* A = static_cast<const Data*>(p->a);
    bool launched = false;
    if constexpr (std::is_same<Data, float>::value) {
      if (!g_test_loss_general && loss_rows_usable(g, scores, A)) {
        rc = fl ? launch_loss_rows<float>(g, scores, A, partials, hist, blocks, info.smem_optin, stream)
                : launch_loss_rows<double>(g, scores, A, partials, hist, blocks, info.smem_optin, stream);
        if (rc) return rc;
        launched = true;
      }
    }
    if (!launched) {
      if (fl) kf<<<blocks, kLossThreads, smem, stream>>>(g, scores, A, partials, hist);
      else kd<<<blocks, kLossThreads, smem, stream>>>(g, scores, A, partials, hist);
    }
    combine_partials_kernel<<<1, 256, 0, stream>>>(partials, blocks, sums);
  }
  hist_to_sums_kernel<<<std::max(1, static_cast<int>((m + 255) / 256)), 256, 0, stream>>>(
      hist, static_cast<int>(m), sums);
  report_gemm_error_kernel<<<1, 32, 0, stream>>>(tc_err, sums);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

}  // namespace sdcab

extern "C" {

int sdcab_objective_from_name(const char* name, double c, double gamma, int64_t k,
                              sdcab_objective* out) {
  return sdcab::objective_from_name(name, c, gamma, k, out);
}

int sdcab_test_set(const char* name, int64_t value) {
  if (!name) return SDCAB_ERR_ARG;
  if (std::strcmp(name, "eval_chunk") == 0) { sdcab::g_test_eval_chunk = value; return SDCAB_OK; }
  if (std::strcmp(name, "gemm_simt") == 0) { sdcab::g_test_force_simt = value ? 1 : 0; return SDCAB_OK; }
  if (std::strcmp(name, "gemm_lose_a_tile") == 0) { sdcab::g_test_lose_a_tile = value ? 1 : 0; return SDCAB_OK; }
  if (std::strcmp(name, "gemm_single_cta") == 0) { sdcab::g_test_single_cta = value ? 1 : 0; return SDCAB_OK; }
  if (std::strcmp(name, "gemm_write_hi") == 0) { sdcab::g_test_write_hi = value ? 1 : 0; return SDCAB_OK; }
  if (std::strcmp(name, "loss_general") == 0) { sdcab::g_test_loss_general = value ? 1 : 0; return SDCAB_OK; }
  if (std::strcmp(name, "gemm_f64_tile") == 0) {
    if (value < 0 || value > 3) return SDCAB_ERR_ARG_RANGE;
    sdcab::set_gemm_f64_tile_mode(static_cast<int>(value));
    return SDCAB_OK;
  }
  if (std::strcmp(name, "primal_simt") == 0) { sdcab::primal_test_force_simt(value ? 1 : 0); return SDCAB_OK; }
  return SDCAB_ERR_ARG;
}

size_t sdcab_eval_workspace_bytes(int64_t n, int64_t m, int64_t elem_size) {
  sdcab::DeviceInfo info;
  int sm = 148;
  if (sdcab::get_device_info(&info) == SDCAB_OK) sm = info.sm_count;
  return sdcab::eval_layout(n, m, elem_size, sm).total;
}

int sdcab_eval_sums_f32_dev(const sdcab_objective* obj, const sdcab_problem* p, double* sums,
                            void* ws, size_t ws_bytes, void* stream) {
  return sdcab::eval_sums_dev<float>(obj, p, sums, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
int sdcab_eval_sums_f64_dev(const sdcab_objective* obj, const sdcab_problem* p, double* sums,
                            void* ws, size_t ws_bytes, void* stream) {
  return sdcab::eval_sums_dev<double>(obj, p, sums, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

int sdcab_eval_finish(const sdcab_objective* obj, int64_t m, const double* sums,
                      sdcab_eval_record* rec, double* accuracy) {
  return sdcab::eval_finish(obj, m, sums, rec, accuracy);
}

int sdcab_eval_f32(const sdcab_objective* obj, const sdcab_problem* hp, sdcab_eval_record* rec,
                   double* accuracy) {
  return sdcab::eval_host<float>(obj, hp, rec, accuracy);
}
int sdcab_eval_f64(const sdcab_objective* obj, const sdcab_problem* hp, sdcab_eval_record* rec,
                   double* accuracy) {
  return sdcab::eval_host<double>(obj, hp, rec, accuracy);
}

int sdcab_eval_sums_fixed_scratch_f32_dev(const sdcab_objective* obj, const sdcab_problem* p,
                                          double* sums, void* stream) {
  return sdcab::eval_sums_fixed_scratch<float>(obj, p, sums, static_cast<cudaStream_t>(stream));
}
int sdcab_eval_sums_fixed_scratch_f64_dev(const sdcab_objective* obj, const sdcab_problem* p,
                                          double* sums, void* stream) {
  return sdcab::eval_sums_fixed_scratch<double>(obj, p, sums, static_cast<cudaStream_t>(stream));
}
size_t sdcab_eval_fixed_scratch_bytes(void) { return sdcab::kFixedScratchBytes; }
const char* sdcab_eval_fixed_scratch_error(void) { return sdcab::g_fixed_scratch_error; }

int sdcab_scores_f32_dev(const sdcab_problem* p, float* scores, void* stream) {
  if (!p || !scores || !p->x) return SDCAB_ERR_ARG;
  void* err = nullptr;
  int rc = sdcab::workspace_reserve(3, 256, &err);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  SDCAB_CUDA_TRY(cudaMemsetAsync(err, 0, sizeof(int), s));
  rc = sdcab::scores_chunk<float>(p, 0, p->n, scores, s, static_cast<int*>(err));
  if (rc) return rc;
  int host_err = 0;
  SDCAB_CUDA_TRY(cudaMemcpyAsync(&host_err, err, sizeof(int), cudaMemcpyDeviceToHost, s));
  SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
  return host_err ? SDCAB_ERR_TIMEOUT : SDCAB_OK;
}
int sdcab_scores_f64_dev(const sdcab_problem* p, double* scores, void* stream) {
  if (!p || !scores || !p->x) return SDCAB_ERR_ARG;
  return sdcab::scores_chunk<double>(p, 0, p->n, scores, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
