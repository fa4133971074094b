// Batched proximal operators: one warp per vector (row of the N x m matrix).
//
// General kernel (any m, any operator): the warp stages its row in shared
// memory with coalesced loads, runs the threshold search of thresholds.cuh on
// it (reductions only, the row is never reordered), then writes
// max(lo, min(map(a - t), hi)) back with coalesced stores.  Algorithmic HBM
// traffic is one read and one write of the matrix.  Rows too long for shared
// memory are read straight from global memory (L2 serves the re-reads).
#include <algorithm>
#include <cstring>

#include "common_host.h"
#include "entropic_rows.cuh"
#include "fast_rows.cuh"
#include "prox_core.cuh"
#include "prox_names.h"
#include "two_simplex_sort.cuh"

namespace sdcab {

constexpr int kRowThreads = 128;  // 4 warps, one row each per iteration

template <typename Data, typename R, int PROX>
__global__ void __launch_bounds__(kRowThreads)
prox_rows_kernel(const Data* a, Data* out, int m, long long n, ProxParams q,
                 sdcab_thresholds* __restrict__ thr_out, int apply, int staged,
                 int m_pad) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  Data* buf = reinterpret_cast<Data*>(smem_raw) + static_cast<size_t>(warp) * m_pad;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + warp;
       row < n; row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const Data* gin = a + row * m;
    Data* g = out + row * m;
    const Data* src = gin;
    if (staged) {
      for (int i = lane; i < m; i += 32) buf[i] = gin[i];
      __syncwarp();
      src = buf;
    }
    if (PROX == kTwoSimplex) {
      StridedRow<Data> ra(src, q.p), rb(src + q.p, m - q.p);
      ThrPair<R> pr = thr_two_simplex<R>(ra, rb, static_cast<R>(q.rhs));
      if (thr_out && lane == 0) {
        sdcab_thresholds o;
        o.reserved = 0;
        o.t = pr.a.t; o.lo = pr.a.lo; o.hi = pr.a.hi; o.num_hi = pr.a.nU; o.num_mid = pr.a.nM;
        o.status = thr_status(pr.a);
        thr_out[2 * row] = o;
        o.t = pr.b.t; o.lo = pr.b.lo; o.hi = pr.b.hi; o.num_hi = pr.b.nU; o.num_mid = pr.b.nM;
        o.status = thr_status(pr.b);
        thr_out[2 * row + 1] = o;
      }
      if (apply) {
        Applier<Data> fa(pr.a, kMapIdentity, 1.0), fb(pr.b, kMapIdentity, 1.0);
        for (int i = lane; i < m; i += 32) g[i] = (i < q.p) ? fa(src[i]) : fb(src[i]);
      }
    } else {
      StridedRow<Data> view(src, m);
      Thr<R> thr = compute_thresholds<R>(PROX, view, q);
      if (thr_out && lane == 0) {
        sdcab_thresholds o;
        o.t = thr.t; o.lo = thr.lo; o.hi = thr.hi; o.num_hi = thr.nU; o.num_mid = thr.nM;
        o.status = thr_status(thr); o.reserved = 0;
        thr_out[row] = o;
      }
      if (apply) {
        Applier<Data> f(thr, prox_map(PROX), q.alpha);
        for (int i = lane; i < m; i += 32) g[i] = f(src[i]);
      }
    }
    __syncwarp();
  }
}

// x <- W(exp(x)), elementwise (include/sdca/prox/proxdef.h:386-400 with
// lambert_w_exp_map, include/sdca/math/functor.h:24-27 of the reference).
template <typename Data>
__global__ void __launch_bounds__(256)
lambert_kernel(const Data* x, Data* y, long long count) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  constexpr int V = 16 / sizeof(Data);
  typedef typename std::conditional<sizeof(Data) == 4, float4, double2>::type Vec;
  const long long nvec = count / V;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (aligned) {
    const Vec* xv = reinterpret_cast<const Vec*>(x);
    Vec* yv = reinterpret_cast<Vec*>(y);
    for (long long j = i; j < nvec; j += stride) {
      Vec v = xv[j];
      Data* e = reinterpret_cast<Data*>(&v);
#pragma unroll
      for (int l = 0; l < V; ++l) e[l] = lambert_w_exp(e[l]);
      yv[j] = v;
    }
    for (long long j = nvec * V + i; j < count; j += stride) y[j] = lambert_w_exp(x[j]);
  } else {
    for (long long j = i; j < count; j += stride) y[j] = lambert_w_exp(x[j]);
  }
}

template <typename Data>
int launch_lambert(const Data* x, Data* y, long long count, cudaStream_t stream) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;
  const int threads = 256;
  long long want = (count / (16 / sizeof(Data)) + threads - 1) / threads;
  int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>(want, 8LL * info.sm_count)));
  lambert_kernel<Data><<<blocks, threads, 0, stream>>>(x, y, count);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

template <typename Data, typename R, int PROX>
int launch_rows(const Data* a, Data* out, int m, long long n, const ProxParams& q,
                sdcab_thresholds* thr_out, int apply, cudaStream_t stream) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;
  auto kernel = prox_rows_kernel<Data, R, PROX>;
  const int warps = kRowThreads / 32;
  const int m_pad = (m + 15) & ~15;
  size_t smem = static_cast<size_t>(warps) * m_pad * sizeof(Data);
  int staged = 1;
  if (smem > info.smem_optin) { staged = 0; smem = 0; }
  if (smem > 48 * 1024) {
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
  }
  int per_sm = 0;
  SDCAB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kRowThreads, smem));
  if (per_sm < 1) per_sm = 1;
  long long want = (n + warps - 1) / warps;
  int blocks = static_cast<int>(std::max<long long>(
      1, std::min<long long>(want, static_cast<long long>(per_sm) * info.sm_count)));
  kernel<<<blocks, kRowThreads, smem, stream>>>(a, out, m, n, q, thr_out, apply, staged, m_pad);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

// Float rows of the entropic projections go to the grouped kernel when the
// launch qualifies (same alignment rules as the register rows).
template <typename R>
int try_entropic_rows(int prox, const float* a, float* out, int m, long long n,
                      const ProxParams& q, cudaStream_t stream) {
  if (m % 4 != 0 || m < 8) return kNoFastPath;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15) return kNoFastPath;
  return launch_entropic_rows<R>(prox, a, out, m, n, q, stream);
}
template <typename R>
int try_entropic_rows(int, const double*, double*, int, long long, const ProxParams&, cudaStream_t) {
  return kNoFastPath;
}

template <typename Data, typename R>
int launch_two_simplex_sort(const Data* a, Data* out, int m, long long n, const ProxParams& q,
                            sdcab_thresholds* thr_out, int apply, cudaStream_t stream) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;
  const int pa = pow2_ceil(q.p), pb = pow2_ceil(m - q.p);
  const int warps = kSortThreads / 32;
  const size_t smem = static_cast<size_t>(warps) * (pa + pb) * sizeof(Data);
  // the sorted copies of both blocks live in shared memory: rows beyond that are refused
  if (smem + 2048 > info.smem_optin) return SDCAB_ERR_TOO_LARGE;
  auto kernel = two_simplex_sort_kernel<Data, R>;
  // the kernel also has about 1 KB of static shared memory, which counts towards the 48 KB
  // that need no opt-in
  if (smem + 2048 > 48 * 1024)
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(smem)));
  const long long want = (n + warps - 1) / warps;
  const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>(want, 8LL * info.sm_count)));
  kernel<<<blocks, kSortThreads, smem, stream>>>(a, out, m, n, q, thr_out, apply, pa, pb);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

template <typename Data, typename R>
int dispatch_prox(int prox, const Data* a, Data* out, int m, long long n, const ProxParams& q,
                  sdcab_thresholds* thr_out, int apply, cudaStream_t stream) {
  if (prox == kTwoSimplexSort)
    return launch_two_simplex_sort<Data, R>(a, out, m, n, q, thr_out, apply, stream);
  // the register-row kernels solve on compacted candidates and have no exact
  // recomputation step: the accurate-math variant takes the general kernel
  if (apply && !thr_out && !q.accurate) {
    int rc = try_entropic_rows<R>(prox, a, out, m, n, q, stream);
    if (rc != kNoFastPath) return rc;
    rc = launch_fast_rows<Data, R>(prox, a, out, m, n, q, stream);
    if (rc != kNoFastPath) return rc;
  }
  switch (prox) {
#define CASE(ID) case ID: return launch_rows<Data, R, ID>(a, out, m, n, q, thr_out, apply, stream);
    CASE(kKnapsackEq) CASE(kKnapsackLe) CASE(kKnapsackLeBiased) CASE(kTopkSimplex)
    CASE(kTopkSimplexBiased) CASE(kTopkCone) CASE(kTopkConeBiased) CASE(kEntropy)
    CASE(kEntropyNorm) CASE(kTopkEntropy) CASE(kTopkEntropyBiased) CASE(kTwoSimplex)
#undef CASE
    default: break;
  }
  return SDCAB_ERR_PROX;
}

// Argument checks of matsdca_prox (src/matlab/mex_prox.cpp:132-136 of the
// reference); p is only checked for the two-block operators so that m == 1
// stays usable for the others.
static int check_args(int prox, long long m, long long n, const sdcab_prox_opts* o) {
  if (!o) return SDCAB_ERR_ARG;
  if (m <= 0 || n <= 0) return SDCAB_ERR_NOT_EMPTY;
  if (m > 0x7fffffffLL) return SDCAB_ERR_TOO_LARGE;
  if (!(o->rhs >= 0) || !(o->rho >= 0) || !(o->alpha > 0)) return SDCAB_ERR_ARG_RANGE;
  if (o->k < 1 || o->k > m) return SDCAB_ERR_ARG_RANGE;
  if ((prox == kTwoSimplex || prox == kTwoSimplexSort) && (o->p < 1 || o->p > m - 1))
    return SDCAB_ERR_ARG_RANGE;
  // two_simplex_sort.h:34: rhs > 0 is a precondition of the sort-based routine
  if (prox == kTwoSimplexSort && !(o->rhs > 0)) return SDCAB_ERR_ARG_RANGE;
  if (o->precision != SDCAB_PRECISION_DOUBLE && o->precision != SDCAB_PRECISION_FLOAT)
    return SDCAB_ERR_PRECISION;
  return SDCAB_OK;
}

template <typename Data>
int prox_dev(const char* name, const Data* a, Data* out, long long m, long long n,
             const sdcab_prox_opts* o, sdcab_thresholds* thr_out, int apply,
             cudaStream_t stream) {
  const int prox = prox_id_from_name(name);
  if (prox < 0) return SDCAB_ERR_PROX;
  if (!a || (apply && !out)) return SDCAB_ERR_ARG;
  int rc = check_args(prox, m, n, o);
  if (rc) return rc;
  if (prox == kLambertWExp) {
    if (thr_out) return SDCAB_ERR_PROX;
    return launch_lambert<Data>(a, out, m * n, stream);
  }
  ProxParams q;
  q.lo = o->lo; q.hi = o->hi; q.rhs = o->rhs; q.rho = o->rho; q.alpha = o->alpha;
  q.k = static_cast<int>(o->k); q.p = static_cast<int>(o->p);
  q.accurate = o->accurate_math ? 1 : 0;
  if (o->precision == SDCAB_PRECISION_FLOAT)
    return dispatch_prox<Data, float>(prox, a, out, static_cast<int>(m), n, q, thr_out, apply, stream);
  return dispatch_prox<Data, double>(prox, a, out, static_cast<int>(m), n, q, thr_out, apply, stream);
}

// Host-buffer form: rows are streamed through two device buffers so that the
// upload of one chunk, the kernel on the previous one and the download of the
// one before overlap on three streams.
template <typename Data>
int prox_host(const char* name, const Data* a, long long m, long long n,
              const sdcab_prox_opts* o, Data* out, sdcab_thresholds* thr) {
  const int prox = prox_id_from_name(name);
  if (prox < 0) return SDCAB_ERR_PROX;
  if (!a) return SDCAB_ERR_ARG;
  int rc = check_args(prox, m, n, o);
  if (rc) return rc;
  const bool want_thr = (thr != nullptr);
  const int per_row_thr = (prox == kTwoSimplex || prox == kTwoSimplexSort) ? 2 : 1;
  const size_t row_bytes = static_cast<size_t>(m) * sizeof(Data);
  // 32 MiB per chunk measured best on PCIe Gen5 (64 MiB: 6 % slower, more of the
  // transfer runs one-directional at the ends; 16 MiB and below: slower again)
  const size_t target = static_cast<size_t>(32) << 20;
  long long rows_per_chunk = std::max<long long>(1, static_cast<long long>(target / row_bytes));
  rows_per_chunk = std::min(rows_per_chunk, n);
  const int kBuf = 3;
  void* dbuf = nullptr; void* tbuf = nullptr;
  // one host-buffer call at a time per device: the scratch and the streams are shared
  std::lock_guard<std::mutex> call_lock(*host_call_mutex());
  rc = workspace_reserve(0, kBuf * rows_per_chunk * row_bytes, &dbuf);
  if (rc) return rc;
  if (want_thr) {
    rc = workspace_reserve(1, kBuf * rows_per_chunk * per_row_thr * sizeof(sdcab_thresholds), &tbuf);
    if (rc) return rc;
  }
  cudaStream_t streams[kBuf];
  rc = pipeline_streams(kBuf, streams);
  if (rc) return rc;
  long long done = 0;
  int slot = 0;
  while (done < n) {
    const long long rows = std::min(rows_per_chunk, n - done);
    cudaStream_t s = streams[slot];
    Data* d = static_cast<Data*>(dbuf) + static_cast<size_t>(slot) * rows_per_chunk * m;
    sdcab_thresholds* dt = want_thr
        ? static_cast<sdcab_thresholds*>(tbuf) + static_cast<size_t>(slot) * rows_per_chunk * per_row_thr
        : nullptr;
    SDCAB_CUDA_TRY(cudaMemcpyAsync(d, a + done * m, rows * row_bytes, cudaMemcpyHostToDevice, s));
    rc = prox_dev<Data>(name, d, d, m, rows, o, dt, want_thr ? 0 : 1, s);
    if (rc) return rc;
    if (want_thr) {
      SDCAB_CUDA_TRY(cudaMemcpyAsync(thr + done * per_row_thr, dt,
                                     rows * per_row_thr * sizeof(sdcab_thresholds),
                                     cudaMemcpyDeviceToHost, s));
    } else {
      SDCAB_CUDA_TRY(cudaMemcpyAsync(out + done * m, d, rows * row_bytes, cudaMemcpyDeviceToHost, s));
    }
    done += rows;
    slot = (slot + 1) % kBuf;
    // a buffer is reused only after the stream that owns it has drained
    if (done < n) SDCAB_CUDA_TRY(cudaStreamSynchronize(streams[slot]));
  }
  for (int i = 0; i < kBuf; ++i) SDCAB_CUDA_TRY(cudaStreamSynchronize(streams[i]));
  return SDCAB_OK;
}

}  // namespace sdcab

extern "C" {

void sdcab_prox_opts_default(sdcab_prox_opts* o) {
  if (!o) return;
  o->lo = 0; o->hi = 1; o->rhs = 1; o->rho = 1; o->alpha = 1;
  o->k = 1; o->p = 1; o->precision = SDCAB_PRECISION_DOUBLE; o->accurate_math = 0;
}

int sdcab_prox_f32_dev(const char* prox, float* a, int64_t m, int64_t n,
                       const sdcab_prox_opts* o, void* stream) {
  return sdcab::prox_dev<float>(prox, a, a, m, n, o, nullptr, 1, static_cast<cudaStream_t>(stream));
}
int sdcab_prox_f64_dev(const char* prox, double* a, int64_t m, int64_t n,
                       const sdcab_prox_opts* o, void* stream) {
  return sdcab::prox_dev<double>(prox, a, a, m, n, o, nullptr, 1, static_cast<cudaStream_t>(stream));
}
int sdcab_prox_to_f32_dev(const char* prox, const float* a, float* out, int64_t m, int64_t n,
                          const sdcab_prox_opts* o, void* stream) {
  return sdcab::prox_dev<float>(prox, a, out, m, n, o, nullptr, 1, static_cast<cudaStream_t>(stream));
}
int sdcab_prox_to_f64_dev(const char* prox, const double* a, double* out, int64_t m, int64_t n,
                          const sdcab_prox_opts* o, void* stream) {
  return sdcab::prox_dev<double>(prox, a, out, m, n, o, nullptr, 1, static_cast<cudaStream_t>(stream));
}
int sdcab_prox_f32(const char* prox, float* a, int64_t m, int64_t n,
                   const sdcab_prox_opts* o, float* out) {
  return sdcab::prox_host<float>(prox, a, m, n, o, out ? out : a, nullptr);
}
int sdcab_prox_f64(const char* prox, double* a, int64_t m, int64_t n,
                   const sdcab_prox_opts* o, double* out) {
  return sdcab::prox_host<double>(prox, a, m, n, o, out ? out : a, nullptr);
}
int sdcab_thresholds_f32_dev(const char* prox, const float* a, int64_t m, int64_t n,
                             const sdcab_prox_opts* o, sdcab_thresholds* thr, void* stream) {
  if (!thr) return SDCAB_ERR_ARG;
  return sdcab::prox_dev<float>(prox, a, nullptr, m, n, o, thr, 0,
                                static_cast<cudaStream_t>(stream));
}
int sdcab_thresholds_f64_dev(const char* prox, const double* a, int64_t m, int64_t n,
                             const sdcab_prox_opts* o, sdcab_thresholds* thr, void* stream) {
  if (!thr) return SDCAB_ERR_ARG;
  return sdcab::prox_dev<double>(prox, a, nullptr, m, n, o, thr, 0,
                                 static_cast<cudaStream_t>(stream));
}
int sdcab_thresholds_f32(const char* prox, const float* a, int64_t m, int64_t n,
                         const sdcab_prox_opts* o, sdcab_thresholds* thr) {
  if (!thr) return SDCAB_ERR_ARG;
  return sdcab::prox_host<float>(prox, a, m, n, o, nullptr, thr);
}
int sdcab_thresholds_f64(const char* prox, const double* a, int64_t m, int64_t n,
                         const sdcab_prox_opts* o, sdcab_thresholds* thr) {
  if (!thr) return SDCAB_ERR_ARG;
  return sdcab::prox_host<double>(prox, a, m, n, o, nullptr, thr);
}
int sdcab_lambert_w_exp_f32_dev(float* x, int64_t count, void* stream) {
  if (!x || count <= 0) return SDCAB_ERR_NOT_EMPTY;
  return sdcab::launch_lambert<float>(x, x, count, static_cast<cudaStream_t>(stream));
}
int sdcab_lambert_w_exp_f64_dev(double* x, int64_t count, void* stream) {
  if (!x || count <= 0) return SDCAB_ERR_NOT_EMPTY;
  return sdcab::launch_lambert<double>(x, x, count, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
