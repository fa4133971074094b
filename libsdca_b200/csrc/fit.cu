// SDCA fit on the device: solver::solve of the reference
// (include/sdca/solver.h:39-117) with update_variables
// (include/sdca/solver/update.h:52-107) as the step.
//
// The steps of an epoch form a sequential chain -- step s reads the dual
// variables step s-1 wrote -- so the unit of parallelism is the inside of one
// step: its score product A K_i (or W'x_i) is spread over every SM, and the
// block that finishes last adds the per-block partial sums in a fixed order and
// runs the objective's update on one warp.  One launch per step, no block ever
// waits for another; the launches of an epoch are replayed from a CUDA graph.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <vector>

#include "common_host.h"
#include "eval_host.h"
#include "fit_host.h"
#include "update_core.cuh"

namespace sdcab {
namespace {

constexpr int kFitThreads = 512;
constexpr int kFitWarps = kFitThreads / 32;
constexpr int kStepsPerGraph = 500;

struct FitState {
  long long step;        // position in the epoch's example order
  unsigned int ticket;   // blocks that have delivered their partial sums
  unsigned int pad;
};

template <typename T> __device__ __forceinline__ T ld_cg(const T* p) { return __ldcg(p); }

// ---- kernel input ------------------------------------------------------------
// scores_j = sum_n A[j + m n] K[n, i]: every warp takes examples n = gw, gw + GW,
// ... and keeps NACC classes per lane; the block adds its warps' sums and stores
// m partial sums; the last block to arrive finishes the step.
template <typename Data, typename R, int NACC>
__global__ void __launch_bounds__(kFitThreads, 1)
fit_step_kernel_input(ObjectiveParams o, const Data* __restrict__ K, Data* A,
                      const int64_t* __restrict__ labels, const int64_t* __restrict__ order,
                      FitState* st, double* partials, int m, long long n) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* red = reinterpret_cast<double*>(smem_raw);              // kFitWarps x tile
  __shared__ bool s_last;
  constexpr int kTile = 32 * NACC;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long i = order[st->step];
  const Data* Ki = K + n * i;
  const Data norm2 = Ki[i];
  const bool active = norm2 > Data(0);   // update.h:97: nothing to do otherwise

  if (active) {
    const long long gw = static_cast<long long>(blockIdx.x) * kFitWarps + warp;
    const long long GW = static_cast<long long>(gridDim.x) * kFitWarps;
    for (int j0 = 0; j0 < m; j0 += kTile) {
      double acc[NACC];
#pragma unroll
      for (int v = 0; v < NACC; ++v) acc[v] = 0.0;
      long long e = gw;
      // four examples in flight per warp
      for (; e + 3 * GW < n; e += 4 * GW) {
        Data a[4][NACC];
        Data kv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const long long ee = e + u * GW;
          kv[u] = Ki[ee];
          const Data* row = A + ee * m + j0;
#pragma unroll
          for (int v = 0; v < NACC; ++v) {
            const int j = lane + 32 * v;
            a[u][v] = (j0 + j < m) ? ld_cg(row + j) : Data(0);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int v = 0; v < NACC; ++v)
            acc[v] = fma(static_cast<double>(a[u][v]), static_cast<double>(kv[u]), acc[v]);
      }
      for (; e < n; e += GW) {
        const Data kv = Ki[e];
        const Data* row = A + e * m + j0;
#pragma unroll
        for (int v = 0; v < NACC; ++v) {
          const int j = lane + 32 * v;
          const Data a = (j0 + j < m) ? ld_cg(row + j) : Data(0);
          acc[v] = fma(static_cast<double>(a), static_cast<double>(kv), acc[v]);
        }
      }
#pragma unroll
      for (int v = 0; v < NACC; ++v) red[warp * kTile + lane + 32 * v] = acc[v];
      __syncthreads();
      for (int j = tid; j < kTile && j0 + j < m; j += kFitThreads) {
        double s = 0.0;
#pragma unroll
        for (int w = 0; w < kFitWarps; ++w) s += red[w * kTile + j];
        partials[static_cast<long long>(blockIdx.x) * m + j0 + j] = s;
      }
      __syncthreads();
    }
  }

  // hand in this block's part; the last one continues
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int t = atomicAdd(&st->ticket, 1u);
    s_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  if (active) {
    Data* scores = reinterpret_cast<Data*>(smem_raw);
    Data* a_s = scores + m;
    Data* v_s = a_s + m;
    Data* a_g = A + i * m;
    const int G = gridDim.x;
    for (int j = tid; j < m; j += kFitThreads) {
      double s = 0.0;
      int g = 0;
      for (; g + 8 <= G; g += 8) {
        double p[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) p[u] = ld_cg(partials + static_cast<long long>(g + u) * m + j);
#pragma unroll
        for (int u = 0; u < 8; ++u) s += p[u];
      }
      for (; g < G; ++g) s += ld_cg(partials + static_cast<long long>(g) * m + j);
      scores[j] = static_cast<Data>(s);
      a_s[j] = a_g[j];
    }
    __syncthreads();
    if (warp == 0) {
      const int y = static_cast<int>(labels[i]);
      update_dual_variables_multiclass<R, Data>(o, norm2, scores, a_s, v_s, m, y);
      for (int j = lane; j < m; j += 32) a_g[j] = a_s[j];
    }
  }
  if (tid == 0) {
    st->ticket = 0;
    st->step += 1;
  }
}

// ---- feature input -------------------------------------------------------------
// scores_j = <W_j, x_i> with W d x m, one warp per class.  The rank-one change of
// W that step s owes (update.h:77-84) is applied by step s+1 while it reads the
// columns anyway: W_j -= x_prev * delta_j, then the dot product with x_i.  A
// last launch with `flush` set applies the change the final step left behind.
struct PendingUpdate {
  long long example;     // -1: nothing pending
  long long pad;
};

template <typename Data, typename R>
__global__ void __launch_bounds__(kFitThreads, 1)
fit_step_feature_input(ObjectiveParams o, const Data* __restrict__ X, Data* W, Data* A,
                       const Data* __restrict__ norms, const int64_t* __restrict__ labels,
                       const int64_t* __restrict__ order, FitState* st, PendingUpdate* pend,
                       Data* delta /* m */, Data* scores_g /* m */, int m, long long d, long long n,
                       int flush) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ bool s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long prev = pend->example;
  const long long i = flush ? -1 : order[st->step];
  const Data norm2 = flush ? Data(0) : norms[i];
  const bool active = norm2 > Data(0);
  const Data* xp = prev >= 0 ? X + d * prev : nullptr;
  const Data* xi = active ? X + d * i : nullptr;

  if (prev >= 0 || active) {
    const int gw = blockIdx.x * kFitWarps + warp;
    const int GW = gridDim.x * kFitWarps;
    for (int j = gw; j < m; j += GW) {
      Data* Wj = W + d * j;
      const Data dj = prev >= 0 ? ld_cg(delta + j) : Data(0);
      double s = 0.0;
      if (prev >= 0 && dj != Data(0)) {
        for (long long r = lane; r < d; r += 32) {
          // W_j <- W_j - x_prev * delta_j, product and difference rounded separately
          const Data w = sub_rn_(Wj[r], mul_rn_(xp[r], dj));
          Wj[r] = w;
          if (active) s = fma(static_cast<double>(w), static_cast<double>(xi[r]), s);
        }
      } else if (active) {
        for (long long r = lane; r < d; r += 32)
          s = fma(static_cast<double>(Wj[r]), static_cast<double>(xi[r]), s);
      }
      if (active) {
        s = warp_sum(s);
        if (lane == 0) scores_g[j] = static_cast<Data>(s);
      }
    }
  }

  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int t = atomicAdd(&st->ticket, 1u);
    s_last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  long long next_pending = -1;
  if (active) {
    Data* scores = reinterpret_cast<Data*>(smem_raw);
    Data* a_s = scores + m;
    Data* v_s = a_s + m;
    Data* old = v_s + m;
    Data* a_g = A + i * m;
    for (int j = tid; j < m; j += kFitThreads) {
      scores[j] = ld_cg(scores_g + j);
      const Data a = a_g[j];
      a_s[j] = a; old[j] = a;
    }
    __syncthreads();
    if (warp == 0) {
      const int y = static_cast<int>(labels[i]);
      update_dual_variables_multiclass<R, Data>(o, norm2, scores, a_s, v_s, m, y);
      // delta = old - new; the primal variables move only if it is not negligible
      Data asum = 0;
      for (int j = lane; j < m; j += 32) {
        const Data dlt = old[j] - a_s[j];
        a_g[j] = a_s[j];
        delta[j] = dlt;
        asum += abs_(dlt);
      }
      asum = warp_sum(asum);
      if (asum > num<Data>::eps()) next_pending = i;
    }
  }
  if (tid == 0) {
    pend->example = next_pending;
    st->ticket = 0;
    if (!flush) st->step += 1;
  }
}

// ||x_i||^2 for every example (solver_scratch::init, data/scratch.h)
template <typename Data>
__global__ void column_norms_kernel(const Data* __restrict__ X, Data* norms, long long d, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  const int lane = threadIdx.x & 31;
  const Data* x = X + d * i;
  double s = 0.0;
  for (long long r = lane; r < d; r += 32) s = fma(static_cast<double>(x[r]), static_cast<double>(x[r]), s);
  s = warp_sum(s);
  if (lane == 0) norms[i] = static_cast<Data>(s);
}

template <typename Data> int eval_sums_call(const sdcab_objective*, const sdcab_problem*, double*, void*);
template <> int eval_sums_call<float>(const sdcab_objective* o, const sdcab_problem* p, double* s, void* st) {
  return sdcab_eval_sums_f32_dev(o, p, s, nullptr, 0, st);
}
template <> int eval_sums_call<double>(const sdcab_objective* o, const sdcab_problem* p, double* s, void* st) {
  return sdcab_eval_sums_f64_dev(o, p, s, nullptr, 0, st);
}

struct DeviceBuffers {
  void* p[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int count = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  ~DeviceBuffers() {
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    for (int i = 0; i < count; ++i) cudaFree(p[i]);
    for (int i = 0; i < 4; ++i) if (ev[i]) cudaEventDestroy(ev[i]);
    if (stream) cudaStreamDestroy(stream);
  }
  int alloc(void** out, size_t bytes) {
    SDCAB_CUDA_TRY(cudaMalloc(out, bytes));
    p[count++] = *out;
    return SDCAB_OK;
  }
};

template <typename Data, typename R>
struct StepLauncher {
  ObjectiveParams o;
  const sdcab_problem* t;
  int grid;
  size_t smem;
  FitState* st;
  int64_t* order;
  double* partials;
  PendingUpdate* pend;
  Data *delta, *scores_g, *norms;

  int launch(cudaStream_t s, int flush) const {
    const int m = static_cast<int>(t->m);
    Data* A = static_cast<Data*>(const_cast<void*>(t->a));
    if (t->input_kind == SDCAB_INPUT_KERNEL) {
      const Data* K = static_cast<const Data*>(t->x);
      if (m <= 32)
        fit_step_kernel_input<Data, R, 1><<<grid, kFitThreads, smem, s>>>(o, K, A, t->labels, order, st, partials, m, t->n);
      else if (m <= 64)
        fit_step_kernel_input<Data, R, 2><<<grid, kFitThreads, smem, s>>>(o, K, A, t->labels, order, st, partials, m, t->n);
      else if (m <= 128)
        fit_step_kernel_input<Data, R, 4><<<grid, kFitThreads, smem, s>>>(o, K, A, t->labels, order, st, partials, m, t->n);
      else
        fit_step_kernel_input<Data, R, 8><<<grid, kFitThreads, smem, s>>>(o, K, A, t->labels, order, st, partials, m, t->n);
    } else {
      fit_step_feature_input<Data, R><<<grid, kFitThreads, smem, s>>>(
          o, static_cast<const Data*>(t->x), static_cast<Data*>(const_cast<void*>(t->w)), A, norms,
          t->labels, order, st, pend, delta, scores_g, m, t->d, t->n, flush);
    }
    SDCAB_CUDA_TRY(cudaGetLastError());
    return SDCAB_OK;
  }

  template <typename F>
  static int set_smem(F* kernel, size_t bytes) {
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(bytes)));
    return SDCAB_OK;
  }
  int prepare() const {
    if (t->input_kind == SDCAB_INPUT_KERNEL) {
      int rc = set_smem(fit_step_kernel_input<Data, R, 1>, smem); if (rc) return rc;
      rc = set_smem(fit_step_kernel_input<Data, R, 2>, smem); if (rc) return rc;
      rc = set_smem(fit_step_kernel_input<Data, R, 4>, smem); if (rc) return rc;
      return set_smem(fit_step_kernel_input<Data, R, 8>, smem);
    }
    return set_smem(fit_step_feature_input<Data, R>, smem);
  }
};

template <typename Data, typename R>
int fit_dev(const sdcab_objective* obj, const sdcab_problem* train, const sdcab_fit_criteria* crit,
            const int64_t* permutations, sdcab_eval_record* evals, int64_t evals_cap,
            sdcab_fit_result* result, cudaStream_t user_stream) {
  const long long n = train->n, m = train->m, d = train->d;
  const bool kernel_input = (train->input_kind == SDCAB_INPUT_KERNEL);
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;

  DeviceBuffers buf;
  SDCAB_CUDA_TRY(cudaStreamCreateWithFlags(&buf.stream, cudaStreamNonBlocking));
  for (int e = 0; e < 4; ++e) SDCAB_CUDA_TRY(cudaEventCreate(&buf.ev[e]));
  cudaStream_t s = buf.stream;
  // everything queued on the caller's stream so far comes first
  SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[0], user_stream));
  SDCAB_CUDA_TRY(cudaStreamWaitEvent(s, buf.ev[0], 0));

  StepLauncher<Data, R> L;
  L.o = to_params(obj);
  L.t = train;
  L.grid = info.sm_count;
  if (!kernel_input) L.grid = static_cast<int>(std::min<long long>(info.sm_count, (m + kFitWarps - 1) / kFitWarps));
  const size_t smem_update = static_cast<size_t>(4 * m) * sizeof(Data);
  const size_t smem_reduce = kernel_input ? static_cast<size_t>(kFitWarps) * 256 * sizeof(double) : 0;
  L.smem = std::max(smem_update, smem_reduce);
  if (L.smem > info.smem_optin) return SDCAB_ERR_TOO_LARGE;
  L.pend = nullptr; L.delta = nullptr; L.scores_g = nullptr; L.norms = nullptr; L.partials = nullptr;

  void* ptr = nullptr;
  rc = buf.alloc(&ptr, sizeof(FitState)); if (rc) return rc;
  L.st = static_cast<FitState*>(ptr);
  rc = buf.alloc(&ptr, static_cast<size_t>(n) * sizeof(long long)); if (rc) return rc;
  L.order = static_cast<int64_t*>(ptr);
  double* sums_dev = nullptr;
  rc = buf.alloc(&ptr, SDCAB_EVAL_SUMS(m) * sizeof(double)); if (rc) return rc;
  sums_dev = static_cast<double*>(ptr);
  if (kernel_input) {
    rc = buf.alloc(&ptr, static_cast<size_t>(L.grid) * m * sizeof(double)); if (rc) return rc;
    L.partials = static_cast<double*>(ptr);
  } else {
    rc = buf.alloc(&ptr, sizeof(PendingUpdate)); if (rc) return rc;
    L.pend = static_cast<PendingUpdate*>(ptr);
    rc = buf.alloc(&ptr, static_cast<size_t>(2 * m + n) * sizeof(Data)); if (rc) return rc;
    L.delta = static_cast<Data*>(ptr);
    L.scores_g = L.delta + m;
    L.norms = L.scores_g + m;
    const PendingUpdate none = {-1, 0};
    SDCAB_CUDA_TRY(cudaMemcpyAsync(L.pend, &none, sizeof(none), cudaMemcpyHostToDevice, s));
    const int wpb = 8;
    column_norms_kernel<Data><<<static_cast<unsigned>((n + wpb - 1) / wpb), wpb * 32, 0, s>>>(
        static_cast<const Data*>(train->x), L.norms, d, n);
    SDCAB_CUDA_TRY(cudaGetLastError());
  }
  rc = L.prepare();
  if (rc) return rc;

  sdcab_problem ep = *train;
  ep.is_train = 1; ep.a_row_offset = 0; ep.include_primal_regularizer = 1;
  std::vector<double> sums(static_cast<size_t>(SDCAB_EVAL_SUMS(m)));
  std::vector<sdcab_eval_record> history;
  double eval_ms = 0, solve_ms = 0;
  auto evaluate = [&]() -> int {
    SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[2], s));
    int erc = eval_sums_call<Data>(obj, &ep, sums_dev, s);
    if (erc) return erc;
    SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[3], s));
    SDCAB_CUDA_TRY(cudaMemcpyAsync(sums.data(), sums_dev, sums.size() * sizeof(double),
                                   cudaMemcpyDeviceToHost, s));
    SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
    float ms = 0;
    SDCAB_CUDA_TRY(cudaEventElapsedTime(&ms, buf.ev[2], buf.ev[3]));
    eval_ms += ms;
    sdcab_eval_record rec;
    erc = eval_finish(obj, m, sums.data(), &rec, nullptr);
    if (erc) return erc;
    history.push_back(rec);
    if (evals && static_cast<int64_t>(history.size()) <= evals_cap) evals[history.size() - 1] = rec;
    return SDCAB_OK;
  };
  const double eps_floor = std::max(
      static_cast<double>(num<Data>::eps()), static_cast<double>(num<R>::eps()));
  auto check = [&](int status, int64_t epoch) {
    const sdcab_eval_record* last = history.empty() ? nullptr : &history.back();
    const sdcab_eval_record* before = history.size() > 1 ? &history[history.size() - 2] : nullptr;
    return check_stopping(status, last, before, crit->epsilon, epoch, crit->max_epoch, eps_floor);
  };

  // begin_solve (solver.h:59-80)
  int64_t epoch = 0;
  int status = (crit->max_epoch > 0) ? SDCAB_FIT_SOLVING : SDCAB_FIT_MAX_EPOCH;
  bool evaluated = false;
  if (crit->eval_on_start) {
    rc = evaluate(); if (rc) return rc;
    status = check(status, epoch);
  }

  MinstdRand gen;
  std::vector<int64_t> order_host(static_cast<size_t>(n));
  for (long long i = 0; i < n; ++i) order_host[static_cast<size_t>(i)] = i;
  const FitState zero_state = {0, 0, 0};
  SDCAB_CUDA_TRY(cudaMemcpyAsync(L.st, &zero_state, sizeof(zero_state), cudaMemcpyHostToDevice, s));

  const long long per_graph = std::min<long long>(kStepsPerGraph, n);
  while (status == SDCAB_FIT_SOLVING) {
    // begin_epoch (solver.h:94-100)
    evaluated = false;
    const int64_t* order_src;
    if (permutations) {
      order_src = permutations + epoch * n;
    } else {
      shuffle_like_libstdcxx(order_host, gen);
      order_src = order_host.data();
    }
    SDCAB_CUDA_TRY(cudaMemcpyAsync(L.order, order_src, static_cast<size_t>(n) * sizeof(long long),
                                   cudaMemcpyHostToDevice, s));
    SDCAB_CUDA_TRY(cudaMemsetAsync(&L.st->step, 0, sizeof(long long), s));
    SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[0], s));
    if (!buf.exec) {
      // per_graph consecutive steps recorded once; every step reads its example
      // from the order array through the device-side step counter, so the same
      // recording serves every stretch of every epoch
      SDCAB_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
      int lrc = SDCAB_OK;
      for (long long k = 0; k < per_graph && lrc == SDCAB_OK; ++k) lrc = L.launch(s, 0);
      cudaError_t cerr = cudaStreamEndCapture(s, &buf.graph);
      if (lrc) return lrc;
      SDCAB_CUDA_TRY(cerr);
      SDCAB_CUDA_TRY(cudaGraphInstantiate(&buf.exec, buf.graph, 0));
    }
    long long done = 0;
    for (; done + per_graph <= n; done += per_graph) SDCAB_CUDA_TRY(cudaGraphLaunch(buf.exec, s));
    for (; done < n; ++done) { rc = L.launch(s, 0); if (rc) return rc; }
    if (!kernel_input) { rc = L.launch(s, 1); if (rc) return rc; }
    SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[1], s));
    SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
    float ms = 0;
    SDCAB_CUDA_TRY(cudaEventElapsedTime(&ms, buf.ev[0], buf.ev[1]));
    solve_ms += ms;

    // end_epoch (solver.h:103-117)
    ++epoch;
    if (crit->eval_epoch > 0 && epoch % crit->eval_epoch == 0) {
      rc = evaluate(); if (rc) return rc;
      evaluated = true;
    }
    status = check(status, epoch);
  }
  // end_solve (solver.h:83-91)
  if (!evaluated && !(crit->eval_on_start && epoch == 0)) {
    rc = evaluate(); if (rc) return rc;
  }
  SDCAB_CUDA_TRY(cudaEventRecord(buf.ev[1], s));
  SDCAB_CUDA_TRY(cudaStreamWaitEvent(user_stream, buf.ev[1], 0));
  SDCAB_CUDA_TRY(cudaStreamSynchronize(s));
  if (result) {
    result->status = status; result->reserved = 0;
    result->epoch = epoch;
    result->num_evals = static_cast<int64_t>(history.size());
    result->solve_seconds = solve_ms * 1e-3;
    result->eval_seconds = eval_ms * 1e-3;
  }
  return SDCAB_OK;
}

int check_fit_args(const sdcab_objective* obj, const sdcab_problem* t, const sdcab_fit_criteria* c) {
  if (!obj || !t || !c) return SDCAB_ERR_ARG;
  if (t->n <= 0 || t->m <= 0 || t->d <= 0) return SDCAB_ERR_NOT_EMPTY;
  if (t->m < 2) return SDCAB_ERR_NUM_DIM;
  if (t->m > 0x7fffffffLL || t->d > 0x7fffffffLL) return SDCAB_ERR_TOO_LARGE;
  int rc = check_objective(obj, t->m);
  if (rc) return rc;
  if (!objective_has_update(obj->id)) return SDCAB_ERR_NOT_IMPLEMENTED;
  if (!t->x || !t->a || !t->labels) return SDCAB_ERR_ARG;
  if (t->input_kind == SDCAB_INPUT_KERNEL) {
    if (t->d != t->n) return SDCAB_ERR_NUM_DIM;
  } else if (t->input_kind == SDCAB_INPUT_FEATURES) {
    if (!t->w) return SDCAB_ERR_ARG;
  } else {
    return SDCAB_ERR_ARG;
  }
  if (!(c->epsilon >= 0) || c->max_epoch < 0 || c->eval_epoch < 0) return SDCAB_ERR_ARG_RANGE;
  return SDCAB_OK;
}

template <typename Data>
int fit_entry(const sdcab_objective* obj, const sdcab_problem* t, const sdcab_fit_criteria* c,
              const int64_t* perm, sdcab_eval_record* evals, int64_t cap, sdcab_fit_result* res,
              void* stream) {
  int rc = check_fit_args(obj, t, c);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (obj->precision == SDCAB_PRECISION_FLOAT)
    return fit_dev<Data, float>(obj, t, c, perm, evals, cap, res, s);
  return fit_dev<Data, double>(obj, t, c, perm, evals, cap, res, s);
}

}  // namespace
}  // namespace sdcab

extern "C" {

int sdcab_epoch_permutations(int64_t n, int64_t num_epochs, int64_t* perm) {
  if (n < 0 || num_epochs < 0 || (!perm && n * num_epochs > 0)) return SDCAB_ERR_ARG;
  sdcab::epoch_permutations(n, num_epochs, perm);
  return SDCAB_OK;
}

int sdcab_fit_f32_dev(const sdcab_objective* obj, const sdcab_problem* train,
                      const sdcab_fit_criteria* criteria, const int64_t* permutations,
                      sdcab_eval_record* evals, int64_t evals_cap, sdcab_fit_result* result,
                      void* stream) {
  return sdcab::fit_entry<float>(obj, train, criteria, permutations, evals, evals_cap, result, stream);
}

int sdcab_fit_f64_dev(const sdcab_objective* obj, const sdcab_problem* train,
                      const sdcab_fit_criteria* criteria, const int64_t* permutations,
                      sdcab_eval_record* evals, int64_t evals_cap, sdcab_fit_result* result,
                      void* stream) {
  return sdcab::fit_entry<double>(obj, train, criteria, permutations, evals, evals_cap, result, stream);
}

}  // extern "C"
