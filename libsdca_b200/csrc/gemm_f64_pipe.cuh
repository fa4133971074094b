// Double-precision score product for few classes: C (M x N) = A (M x K) * op(B) on the
// FP64 tensor cores (mma.sync m8n8k4) with a column tile of 8 * NF columns (NF = 13:
// 104 columns, which m = 100 fills to 96 % where a 128-wide tile is a fifth padding)
// and the operands staged by cp.async three tiles deep, so no warp holds the next tile
// in registers and no barrier waits for a global load issued just before it.
//
// Same operand forms and extras as gemm_kernel (gemm_blocked.cuh): B with the
// contraction index contiguous (scores = X' W) or as its row index (scores = K' A'),
// row gather lists, a split of the contraction index into slices, and rows of B left
// out by owner.  A warp owns 16 rows x all 8 * NF columns of the block's tile: per step of
// four contraction indices it loads 2 + NF fragments for 2 * NF products.
//
// Shared-memory layouts are the global ones (no transposition, which cp.async cannot
// do): a tile with the contraction index contiguous is [row][16 + 4], one with the
// column index contiguous is [k][8 * NF + 4]; with a row length of 4 or 12 (mod 16)
// doubles the fragment loads (lane -> row lane / 4 | k lane % 4, or the transpose) touch
// sixteen different 8-byte banks per half warp.
#pragma once

#include <cstdint>

#include "common_host.h"
// included by gemm_blocked.cuh after mma_f64 and GemmExtras, which it uses

namespace sdcab {
namespace f64pipe {

constexpr int kBK = 16;
constexpr int kStages = 3;
constexpr int kRowK = kBK + 4;          // doubles per staged row, contraction index contiguous

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16- and 8-byte asynchronous copies; bytes past src_bytes are filled with zeros
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" :: "r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// Two consecutive doubles of one row: `valid` of them (0, 1 or 2) lie inside the matrix.
__device__ __forceinline__ void copy_pair(uint32_t dst, const double* src, const double* safe,
                                          int valid, int vec_ok) {
  if (vec_ok) {
    cp_async16(dst, valid ? src : safe, valid * 8);
  } else {
    cp_async8(dst, valid >= 1 ? src : safe, valid >= 1 ? 8 : 0);
    cp_async8(dst + 8, valid >= 2 ? src + 1 : safe, valid >= 2 ? 8 : 0);
  }
}

template <int BM, int NF, bool B_KMAJOR>
struct Shape {
  static constexpr int BN = 8 * NF;
  static constexpr int kThreads = (BM / 16) * 32;
  static constexpr int kRowN = BN + 4;      // doubles per staged row, column index contiguous
  static constexpr int kADoubles = BM * kRowK;
  static constexpr int kBDoubles = B_KMAJOR ? BN * kRowK : kBK * kRowN;
  static constexpr int kStageDoubles = kADoubles + kBDoubles;
  static constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageDoubles * sizeof(double);
};

template <int BM, int NF, bool B_KMAJOR>
__global__ void __launch_bounds__((BM / 16) * 32, BM == 64 ? 3 : 1)
gemm_f64_pipe_kernel(const double* __restrict__ A, const double* __restrict__ B, double* __restrict__ C,
                     int M, int N, int K, long long lda, long long ldb, long long ldc, int a_vec,
                     int b_vec, int c_vec, const int64_t* __restrict__ a_gather,
                     const int64_t* __restrict__ b_gather, int k_per_slice, long long c_slice_stride,
                     const int* __restrict__ k_owner, int skip_owner) {
  typedef Shape<BM, NF, B_KMAJOR> S;
  constexpr int NT = S::kThreads, BN = S::BN, ROWN = S::kRowN;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* smem = reinterpret_cast<double*>(smem_raw);
  const int tid = threadIdx.x;
  const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
  {
    const long long kb = static_cast<long long>(blockIdx.z) * k_per_slice;
    A += kb;
    B += B_KMAJOR ? kb : kb * ldb;
    if (k_owner) k_owner += kb;
    C += static_cast<long long>(blockIdx.z) * c_slice_stride;
    K = (K - kb < k_per_slice) ? static_cast<int>(K - kb) : k_per_slice;
    if (K < 0) K = 0;
  }

  // ---- the copies of one tile.  A pair is two doubles (16 bytes).
  constexpr int A_PAIRS = BM * (kBK / 2);
  constexpr int A_PER = (A_PAIRS + NT - 1) / NT;
  const double* a_rows[A_PER];            // this thread's rows of A are the same for every tile
  unsigned a_ok = 0, b_ok = 0;
#pragma unroll
  for (int it = 0; it < A_PER; ++it) {
    const int idx = tid + it * NT;
    const int r = row0 + idx / (kBK / 2);
    const bool ok = idx < A_PAIRS && r < M;
    // rows outside the matrix point at its start and are copied with zero valid bytes
    a_rows[it] = ok ? A + (a_gather ? static_cast<long long>(a_gather[r]) : r) * lda : A;
    a_ok |= (ok ? 1u : 0u) << it;
  }
  constexpr int BK_PAIRS = B_KMAJOR ? BN * (kBK / 2) : kBK * (BN / 2);
  constexpr int B_PER = (BK_PAIRS + NT - 1) / NT;
  const double* b_rows[B_KMAJOR ? B_PER : 1];
  (void)b_ok; (void)b_rows;
  if constexpr (B_KMAJOR) {
#pragma unroll
    for (int it = 0; it < B_PER; ++it) {
      const int idx = tid + it * NT;
      const int r = col0 + idx / (kBK / 2);
      const bool ok = idx < BK_PAIRS && r < N;
      b_rows[it] = ok ? B + (b_gather ? static_cast<long long>(b_gather[r]) : r) * ldb : B;
      b_ok |= (ok ? 1u : 0u) << it;
    }
  }

  auto load_tile = [&](int kt, int stage) {
    double* As = smem + static_cast<size_t>(stage) * S::kStageDoubles;
    double* Bs = As + S::kADoubles;
    const int k0 = kt * kBK;
#pragma unroll
    for (int it = 0; it < A_PER; ++it) {
      const int idx = tid + it * NT;
      if (A_PAIRS % NT != 0 && idx >= A_PAIRS) break;
      const int r = idx / (kBK / 2), kk = (idx % (kBK / 2)) * 2;
      const int left = K - (k0 + kk);
      const int valid = ((a_ok >> it) & 1u) ? (left >= 2 ? 2 : (left > 0 ? left : 0)) : 0;
      copy_pair(smem_addr(As + r * kRowK + kk), a_rows[it] + k0 + kk, A, valid, a_vec);
    }
    if constexpr (B_KMAJOR) {
#pragma unroll
      for (int it = 0; it < B_PER; ++it) {
        const int idx = tid + it * NT;
        if (BK_PAIRS % NT != 0 && idx >= BK_PAIRS) break;
        const int r = idx / (kBK / 2), kk = (idx % (kBK / 2)) * 2;
        const int left = K - (k0 + kk);
        const int valid = ((b_ok >> it) & 1u) ? (left >= 2 ? 2 : (left > 0 ? left : 0)) : 0;
        copy_pair(smem_addr(Bs + r * kRowK + kk), b_rows[it] + k0 + kk, B, valid, b_vec);
      }
    } else {
#pragma unroll
      for (int it = 0; it < B_PER; ++it) {
        const int idx = tid + it * NT;
        if (BK_PAIRS % NT != 0 && idx >= BK_PAIRS) break;
        const int kk = idx / (BN / 2), nn = (idx % (BN / 2)) * 2;
        const int gk = k0 + kk, gn = col0 + nn;
        // rows of B whose owner is being rewritten elsewhere count as zero and are not read
        const bool row_ok = gk < K && !(k_owner && k_owner[gk] == skip_owner);
        const int left = N - gn;
        const int valid = row_ok ? (left >= 2 ? 2 : (left > 0 ? left : 0)) : 0;
        copy_pair(smem_addr(Bs + kk * ROWN + nn), B + static_cast<long long>(gk) * ldb + gn, B, valid, b_vec);
      }
    }
  };

  const int warp = tid >> 5, lane = tid & 31;
  const int wm = warp * 16;
  const int fr = lane >> 2, fc = lane & 3;
  double acc[2][NF][2];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < NF; ++j) { acc[i][j][0] = 0.0; acc[i][j][1] = 0.0; }

  const int ktiles = (K + kBK - 1) / kBK;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (s < ktiles) load_tile(s, s);
    cp_async_commit();
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    cp_async_wait<kStages - 2>();
    __syncthreads();
    // the stage read in the previous iteration is free now: every warp has passed the barrier
    if (kt + kStages - 1 < ktiles) load_tile(kt + kStages - 1, (kt + kStages - 1) % kStages);
    cp_async_commit();
    const double* As = smem + static_cast<size_t>(kt % kStages) * S::kStageDoubles;
    const double* Bs = As + S::kADoubles;
#pragma unroll
    for (int k4 = 0; k4 < kBK; k4 += 4) {
      const double a0 = As[(wm + fr) * kRowK + k4 + fc];
      const double a1 = As[(wm + 8 + fr) * kRowK + k4 + fc];
#pragma unroll
      for (int j = 0; j < NF; ++j) {
        const double b = B_KMAJOR ? Bs[(j * 8 + fr) * kRowK + k4 + fc] : Bs[(k4 + fc) * ROWN + j * 8 + fr];
        mma_f64(acc[0][j][0], acc[0][j][1], a0, b);
        mma_f64(acc[1][j][0], acc[1][j][1], a1, b);
      }
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = row0 + wm + i * 8 + fr;
    if (r >= M) continue;
#pragma unroll
    for (int j = 0; j < NF; ++j) {
      const int c0 = col0 + j * 8 + 2 * fc;
      double* dst = C + static_cast<long long>(r) * ldc + c0;
      if (c_vec && c0 + 2 <= N) {
        *reinterpret_cast<double2*>(dst) = make_double2(acc[i][j][0], acc[i][j][1]);
      } else {
        if (c0 < N) dst[0] = acc[i][j][0];
        if (c0 + 1 < N) dst[1] = acc[i][j][1];
      }
    }
  }
}

template <int BM, int NF>
int launch(const double* A, const double* B, double* C, int M, int N, int K, long long lda,
           long long ldb, long long ldc, bool b_kmajor, cudaStream_t stream, const GemmExtras& x) {
  auto aligned = [&](const void* p, long long ld) {
    return ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && ld % 2 == 0) ? 1 : 0;
  };
  int k_per_slice = (K + x.slices - 1) / x.slices;
  k_per_slice = (k_per_slice + kBK - 1) / kBK * kBK;
  if (k_per_slice <= 0) k_per_slice = kBK;
  const int a_vec = aligned(A, lda), c_vec = aligned(C, ldc) && (x.c_slice_stride % 2 == 0);
  const int b_vec = aligned(B, ldb);
  constexpr int BN = 8 * NF;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, x.slices);
  if (b_kmajor) {
    typedef Shape<BM, NF, true> S;
    auto kernel = gemm_f64_pipe_kernel<BM, NF, true>;
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(S::kSmemBytes)));
    kernel<<<grid, S::kThreads, S::kSmemBytes, stream>>>(
        A, B, C, M, N, K, lda, ldb, ldc, a_vec, b_vec, c_vec, x.a_gather, x.b_gather, k_per_slice,
        x.c_slice_stride, nullptr, -1);
  } else {
    typedef Shape<BM, NF, false> S;
    auto kernel = gemm_f64_pipe_kernel<BM, NF, false>;
    SDCAB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(S::kSmemBytes)));
    kernel<<<grid, S::kThreads, S::kSmemBytes, stream>>>(
        A, B, C, M, N, K, lda, ldb, ldc, a_vec, b_vec, c_vec, x.a_gather, nullptr, k_per_slice,
        x.c_slice_stride, x.k_owner, x.skip_owner);
  }
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

}  // namespace f64pipe
}  // namespace sdcab
