// Primal variables from dual variables, W = [W0 +] X A'.
//
// Both operands have the contraction index (the example) as their slow index:
// example n holds d contiguous features and m contiguous dual variables.  That is
// the natural layout of an outer-product GEMM: a stage of BK examples is BK rows
// of A and BK rows of X, loaded as they lie in memory, and every thread adds
// a[j] * x[i] for its TJ x TI block of W.  FMA in the data type, like the BLAS
// gemm the reference calls (include/sdca/solver/eval/core.h:164-174).
//
// Float data of more than a few thousand examples goes to the tensor cores instead:
// the paired-CTA 3xTF32 kernel of gemm_pair.cuh in its MN-major form, one pair of CTAs
// per 256 x 256 tile of W walking over all examples in order (a fixed summation order,
// so the result is the same from run to run).
#include <algorithm>
#include <cstdint>

#include "../../include/sdca_b200.h"
#include "common_host.h"
#include "gemm_pair.cuh"
#include "primal.h"

namespace sdcab {

constexpr int kPrimalBJ = 64, kPrimalBI = 128, kPrimalBK = 16, kPrimalTJ = 4, kPrimalTI = 8;
constexpr int kPrimalThreads = (kPrimalBJ / kPrimalTJ) * (kPrimalBI / kPrimalTI);

// blockIdx.x: tile of features, blockIdx.y: tile of classes, blockIdx.z: slice of
// examples.  With one slice the block writes w = w0 + sum; otherwise its partial
// sum goes to slices[z] and primal_reduce_kernel adds the slices up.
template <typename T>
__global__ void __launch_bounds__(kPrimalThreads)
primal_from_dual_kernel(const T* __restrict__ x, const T* __restrict__ a, const T* __restrict__ w0,
                        T* __restrict__ w, T* __restrict__ slices, long long d, long long m,
                        long long n, long long n_per_slice) {
  __shared__ __align__(16) T as[kPrimalBK][kPrimalBJ];
  __shared__ __align__(16) T xs[kPrimalBK][kPrimalBI];
  const int tid = threadIdx.x;
  const int ti = tid % (kPrimalBI / kPrimalTI), tj = tid / (kPrimalBI / kPrimalTI);
  const long long i0 = static_cast<long long>(blockIdx.x) * kPrimalBI;
  const long long j0 = static_cast<long long>(blockIdx.y) * kPrimalBJ;
  const long long k_begin = static_cast<long long>(blockIdx.z) * n_per_slice;
  const long long k_end = min(n, k_begin + n_per_slice);
  T acc[kPrimalTJ][kPrimalTI];
#pragma unroll
  for (int r = 0; r < kPrimalTJ; ++r)
#pragma unroll
    for (int c = 0; c < kPrimalTI; ++c) acc[r][c] = T(0);
  for (long long k0 = k_begin; k0 < k_end; k0 += kPrimalBK) {
#pragma unroll
    for (int it = 0; it < kPrimalBK * kPrimalBJ / kPrimalThreads; ++it) {
      const int idx = tid + it * kPrimalThreads;
      const int kk = idx / kPrimalBJ, jj = idx % kPrimalBJ;
      const bool ok = k0 + kk < k_end && j0 + jj < m;
      as[kk][jj] = ok ? a[(k0 + kk) * m + j0 + jj] : T(0);
    }
#pragma unroll
    for (int it = 0; it < kPrimalBK * kPrimalBI / kPrimalThreads; ++it) {
      const int idx = tid + it * kPrimalThreads;
      const int kk = idx / kPrimalBI, ii = idx % kPrimalBI;
      const bool ok = k0 + kk < k_end && i0 + ii < d;
      xs[kk][ii] = ok ? x[(k0 + kk) * d + i0 + ii] : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kPrimalBK; ++kk) {
      T av[kPrimalTJ], xv[kPrimalTI];
#pragma unroll
      for (int r = 0; r < kPrimalTJ; ++r) av[r] = as[kk][tj * kPrimalTJ + r];
#pragma unroll
      for (int c = 0; c < kPrimalTI; ++c) xv[c] = xs[kk][ti * kPrimalTI + c];
#pragma unroll
      for (int r = 0; r < kPrimalTJ; ++r)
#pragma unroll
        for (int c = 0; c < kPrimalTI; ++c) acc[r][c] = fma(av[r], xv[c], acc[r][c]);
    }
    __syncthreads();
  }
  T* dst = slices ? slices + static_cast<long long>(blockIdx.z) * d * m : w;
#pragma unroll
  for (int r = 0; r < kPrimalTJ; ++r) {
    const long long j = j0 + tj * kPrimalTJ + r;
    if (j >= m) continue;
#pragma unroll
    for (int c = 0; c < kPrimalTI; ++c) {
      const long long i = i0 + ti * kPrimalTI + c;
      if (i >= d) continue;
      const T base = (!slices && w0) ? w0[j * d + i] : T(0);
      dst[j * d + i] = base + acc[r][c];
    }
  }
}

template <typename T>
__global__ void primal_reduce_kernel(const T* __restrict__ slices, const T* __restrict__ w0,
                                     T* __restrict__ w, long long elems, int num_slices) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; e < elems;
       e += stride) {
    T s = w0 ? w0[e] : T(0);
    for (int z = 0; z < num_slices; ++z) s += slices[static_cast<long long>(z) * elems + e];
    w[e] = s;
  }
}

static int g_primal_force_simt = 0;
void primal_test_force_simt(int on) { g_primal_force_simt = on ? 1 : 0; }

// The tensor-core form; kNotTaken when the operands do not qualify.
constexpr int kNotTaken = 1;
inline int primal_tc(const float* x, const float* a, const float* w0, float* w, long long d, long long m,
                     long long n, cudaStream_t stream) {
  if (g_primal_force_simt || n < 2048 || d > 0x7fffffffLL || m > 0x7fffffffLL) return kNotTaken;
  if (!tc2::usable_mn(a, x, w0, m, d) || (d % 4) != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0)
    return kNotTaken;
  void* err = nullptr;
  int rc = workspace_reserve(5, 256, &err);
  if (rc) return rc;
  SDCAB_CUDA_TRY(cudaMemsetAsync(err, 0, sizeof(int), stream));
  rc = tc2::launch_mn(a, x, w0, w, static_cast<int>(m), static_cast<int>(d), n, m, d, d,
                      static_cast<int*>(err), stream);
  if (rc == SDCAB_ERR_NOT_IMPLEMENTED) return kNotTaken;
  if (rc) return rc;
  // a wait that ran out inside the kernel becomes this call's status
  int host_err = 0;
  SDCAB_CUDA_TRY(cudaMemcpyAsync(&host_err, err, sizeof(int), cudaMemcpyDeviceToHost, stream));
  SDCAB_CUDA_TRY(cudaStreamSynchronize(stream));
  return host_err ? SDCAB_ERR_TIMEOUT : SDCAB_OK;
}
inline int primal_tc(const double*, const double*, const double*, double*, long long, long long, long long,
                     cudaStream_t) {
  return kNotTaken;
}

template <typename Data>
int primal_from_dual_dev(const Data* x, const Data* a, const Data* w0, Data* w, long long d,
                         long long m, long long n, cudaStream_t stream) {
  if (!x || !a || !w) return SDCAB_ERR_ARG;
  if (d <= 0 || m <= 0 || n <= 0) return SDCAB_ERR_NOT_EMPTY;
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;
  rc = primal_tc(x, a, w0, w, d, m, n, stream);
  if (rc != kNotTaken) return rc;
  const long long tiles_i = (d + kPrimalBI - 1) / kPrimalBI, tiles_j = (m + kPrimalBJ - 1) / kPrimalBJ;
  if (tiles_i > 0x7fffffffLL || tiles_j > 65535) return SDCAB_ERR_TOO_LARGE;
  // few tiles: slices of examples fill the device
  long long num_slices = 1;
  const long long tiles = tiles_i * tiles_j;
  if (tiles < info.sm_count) {
    num_slices = (2LL * info.sm_count + tiles - 1) / tiles;
    num_slices = std::min<long long>(num_slices, (n + 4 * kPrimalBK - 1) / (4 * kPrimalBK));
    num_slices = std::max<long long>(1, std::min<long long>(num_slices, 64));
  }
  long long n_per_slice = (n + num_slices - 1) / num_slices;
  n_per_slice = (n_per_slice + kPrimalBK - 1) / kPrimalBK * kPrimalBK;
  num_slices = (n + n_per_slice - 1) / n_per_slice;
  Data* slices = nullptr;
  if (num_slices > 1)
    SDCAB_CUDA_TRY(cudaMallocAsync(reinterpret_cast<void**>(&slices),
                                   static_cast<size_t>(num_slices) * d * m * sizeof(Data), stream));
  const dim3 grid(static_cast<unsigned>(tiles_i), static_cast<unsigned>(tiles_j),
                  static_cast<unsigned>(num_slices));
  primal_from_dual_kernel<Data><<<grid, kPrimalThreads, 0, stream>>>(x, a, w0, w, slices, d, m, n,
                                                                    n_per_slice);
  SDCAB_CUDA_TRY(cudaGetLastError());
  if (slices) {
    const long long elems = d * m;
    const int blocks = static_cast<int>(std::max<long long>(
        1, std::min<long long>((elems + 255) / 256, 8LL * info.sm_count)));
    primal_reduce_kernel<Data><<<blocks, 256, 0, stream>>>(slices, w0, w, elems,
                                                           static_cast<int>(num_slices));
    SDCAB_CUDA_TRY(cudaGetLastError());
    SDCAB_CUDA_TRY(cudaFreeAsync(slices, stream));
  }
  return SDCAB_OK;
}

template int primal_from_dual_dev<float>(const float*, const float*, const float*, float*, long long,
                                         long long, long long, cudaStream_t);
template int primal_from_dual_dev<double>(const double*, const double*, const double*, double*,
                                          long long, long long, long long, cudaStream_t);

}  // namespace sdcab

extern "C" {

int sdcab_primal_from_dual_f32_dev(const float* x, const float* a, const float* w0, float* w,
                                   int64_t d, int64_t m, int64_t n, void* stream) {
  return sdcab::primal_from_dual_dev<float>(x, a, w0, w, d, m, n, static_cast<cudaStream_t>(stream));
}
int sdcab_primal_from_dual_f64_dev(const double* x, const double* a, const double* w0, double* w,
                                   int64_t d, int64_t m, int64_t n, void* stream) {
  return sdcab::primal_from_dual_dev<double>(x, a, w0, w, d, m, n, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
