// Blocked GEMM for the score products in the data type: the evaluation's batched
// scores and the fit's per-block scores.  Doubles run on the FP64 tensor cores
// (mma.sync m8n8k4), floats that the tcgen05 kernel cannot take on FMA; both share
// the tile loads with their gathers, slices and masks.
#pragma once

#include <cstdint>
#include <type_traits>

#include "common_host.h"

namespace sdcab {

// ------------------------------------------------------------------ GEMM ----
// C (M x N, row major) = A (M x K, row major) * op(B), with
//   B_KMAJOR:  B is N x K row major  (C = A B')   -- scores = X' W
//   otherwise: B is K x N row major  (C = A B)    -- scores = K' A'
// Thread block tile BM x BN x BK, TM x TN outputs per thread, register
// prefetch of the next tile while the current one is consumed from shared
// memory.  Arithmetic is plain FMA in the data type, accumulating over the
// contraction index in increasing order, like a reference BLAS gemv.
template <typename T> struct Vec16;
template <> struct Vec16<float> { typedef float4 type; };
template <> struct Vec16<double> { typedef double2 type; };

// Loads this thread's share of a rows x BK tile whose contraction index is
// contiguous in memory (16-byte vectors where alignment allows, zero fill past
// the edges).
template <typename T, int BK, int NT, int PER>
__device__ __forceinline__ void load_kmajor_tile(const T* __restrict__ base, long long ld,
                                                 int rows_total, int K, int r0, int k0,
                                                 int vec_ok, int tid, T (&dst)[PER][16 / sizeof(T)],
                                                 const int64_t* __restrict__ gather = nullptr) {
  constexpr int V = 16 / sizeof(T);
  typedef typename Vec16<T>::type Vec;
#pragma unroll
  for (int it = 0; it < PER; ++it) {
    const int idx = tid + it * NT;
    const int r = idx / (BK / V), kv = (idx % (BK / V)) * V;
    const int gk = k0 + kv;
    const bool row_ok = r0 + r < rows_total;
    // row r of the operand is row gather[r] of the matrix when a gather list is given
    const long long gr = row_ok ? (gather ? static_cast<long long>(gather[r0 + r]) : r0 + r) : 0;
    if (row_ok && vec_ok && gk + V <= K) {
      const Vec v = *reinterpret_cast<const Vec*>(base + gr * ld + gk);
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int c = 0; c < V; ++c) dst[it][c] = e[c];
    } else {
#pragma unroll
      for (int c = 0; c < V; ++c)
        dst[it][c] = (row_ok && gk + c < K) ? base[gr * ld + gk + c] : T(0);
    }
  }
}

// FP64 tensor-core product of one 8x4 by 4x8 pair of fragments into an 8x8
// accumulator (mma.sync m8n8k4): lane l holds A[l / 4][l % 4], B[l % 4][l / 4] and
// the accumulator entries [l / 4][2 (l % 4)], [l / 4][2 (l % 4) + 1].
__device__ __forceinline__ void mma_f64(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
               : "+d"(c0), "+d"(c1) : "d"(a), "d"(b));
}

// MMA (double only): the tile product runs on the FP64 tensor cores.  Warps tile
// the block in 32x32 pieces (4x4 fragments each), so the thread count is
// BM * BN / 32 and TM * TN must be 32; everything around the product -- loads,
// gathers, slices, masks, edges -- is shared with the FMA form.
template <typename T, int BM, int BN, int BK, int TM, int TN, bool B_KMAJOR, bool MMA = false>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C, int M, int N,
            int K, long long lda, long long ldb, long long ldc, int a_vec, int b_vec, int c_vec,
            const int64_t* __restrict__ a_gather, const int64_t* __restrict__ b_gather,
            int k_per_slice, long long c_slice_stride, const int* __restrict__ k_owner,
            int skip_owner) {
  constexpr int NT = (BM / TM) * (BN / TN);
  constexpr int V = 16 / sizeof(T);
  // fragment loads of the MMA form are conflict free when a row of the staged
  // tile is 4 (mod 16) doubles long
  constexpr int PAD = MMA ? 4 : V;
  static_assert(!MMA || (sizeof(T) == 8 && TM * TN == 32 && BM % 32 == 0 && BN % 32 == 0 && BK % 4 == 0),
                "the tensor-core form is for double and 32x32 warp tiles");
  typedef typename Vec16<T>::type Vec;
  __shared__ __align__(16) T As[2][BK][BM + PAD];
  __shared__ __align__(16) T Bs[2][BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
  // slice blockIdx.z of the contraction index: a partial product of its own
  {
    const long long kb = static_cast<long long>(blockIdx.z) * k_per_slice;
    A += kb;
    B += B_KMAJOR ? kb : kb * ldb;
    if (k_owner) k_owner += kb;
    C += static_cast<long long>(blockIdx.z) * c_slice_stride;
    K = (K - kb < k_per_slice) ? static_cast<int>(K - kb) : k_per_slice;
    if (K < 0) K = 0;
  }

  constexpr int A_PER = (BM * BK / V) / NT;
  constexpr int B_PER = (BN * BK / V) / NT;
  static_assert(A_PER >= 1 && B_PER >= 1, "tile too small for the thread count");
  T ra[A_PER][V], rb[B_PER][V];

  auto load_b_nmajor = [&](int k0) {
#pragma unroll
    for (int it = 0; it < B_PER; ++it) {
      const int idx = tid + it * NT;
      const int kk = idx / (BN / V), nv = (idx % (BN / V)) * V;
      const int gk = k0 + kk, gn = col0 + nv;
      // rows of B whose owner is being rewritten elsewhere count as zero and are not read
      const bool skipped = k_owner && gk < K && k_owner[gk] == skip_owner;
      if (skipped) {
#pragma unroll
        for (int c = 0; c < V; ++c) rb[it][c] = T(0);
      } else if (gk < K && b_vec && gn + V <= N) {
        const Vec v = *reinterpret_cast<const Vec*>(B + static_cast<long long>(gk) * ldb + gn);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int c = 0; c < V; ++c) rb[it][c] = e[c];
      } else {
#pragma unroll
        for (int c = 0; c < V; ++c)
          rb[it][c] = (gk < K && gn + c < N) ? B[static_cast<long long>(gk) * ldb + gn + c] : T(0);
      }
    }
  };
  auto store_tiles = [&](int buf) {
#pragma unroll
    for (int it = 0; it < A_PER; ++it) {
      const int idx = tid + it * NT;
      const int r = idx / (BK / V), kv = (idx % (BK / V)) * V;
#pragma unroll
      for (int c = 0; c < V; ++c) As[buf][kv + c][r] = ra[it][c];
    }
#pragma unroll
    for (int it = 0; it < B_PER; ++it) {
      const int idx = tid + it * NT;
      if (B_KMAJOR) {
        const int r = idx / (BK / V), kv = (idx % (BK / V)) * V;
#pragma unroll
        for (int c = 0; c < V; ++c) Bs[buf][kv + c][r] = rb[it][c];
      } else {
        const int kk = idx / (BN / V), nv = (idx % (BN / V)) * V;
#pragma unroll
        for (int c = 0; c < V; ++c) Bs[buf][kk][nv + c] = rb[it][c];
      }
    }
  };
  auto load_tiles = [&](int k0) {
    load_kmajor_tile<T, BK, NT, A_PER>(A, lda, M, K, row0, k0, a_vec, tid, ra, a_gather);
    if (B_KMAJOR) load_kmajor_tile<T, BK, NT, B_PER>(B, ldb, N, K, col0, k0, b_vec, tid, rb, b_gather);
    else load_b_nmajor(k0);
  };

  if constexpr (MMA) {
    const int warp = tid >> 5, lane = tid & 31;
    constexpr int WN = BN / 32;
    const int wm = (warp / WN) * 32, wn = (warp % WN) * 32;
    const int fr = lane >> 2, fc = lane & 3;
    double acc2[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc2[i][j][0] = 0.0; acc2[i][j][1] = 0.0; }
    load_tiles(0);
    store_tiles(0);
    __syncthreads();
    const int ktiles = (K + BK - 1) / BK;
    for (int kt = 0; kt < ktiles; ++kt) {
      const int buf = kt & 1;
      if (kt + 1 < ktiles) load_tiles((kt + 1) * BK);
#pragma unroll
      for (int k4 = 0; k4 < BK; k4 += 4) {
        double a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[buf][k4 + fc][wm + i * 8 + fr];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[buf][k4 + fc][wn + j * 8 + fr];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_f64(acc2[i][j][0], acc2[i][j][1], a[i], b[j]);
      }
      if (kt + 1 < ktiles) {
        store_tiles(buf ^ 1);
        __syncthreads();
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = row0 + wm + i * 8 + fr;
      if (r >= M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c0 = col0 + wn + j * 8 + 2 * fc;
        T* dst = C + static_cast<long long>(r) * ldc + c0;
        if (c_vec && c0 + 2 <= N) {
          *reinterpret_cast<double2*>(dst) = make_double2(acc2[i][j][0], acc2[i][j][1]);
        } else {
          if (c0 < N) dst[0] = static_cast<T>(acc2[i][j][0]);
          if (c0 + 1 < N) dst[1] = static_cast<T>(acc2[i][j][1]);
        }
      }
    }
    return;
  }

  T acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = T(0);

  constexpr int HM = TM / 2, HN = TN / 2;  // each thread owns two strips per dimension
  load_tiles(0);
  store_tiles(0);
  __syncthreads();
  const int ktiles = (K + BK - 1) / BK;
  for (int kt = 0; kt < ktiles; ++kt) {
    const int buf = kt & 1;
    if (kt + 1 < ktiles) load_tiles((kt + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      T a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < HM; ++i) {
        a[i] = As[buf][kk][ty * HM + i];
        a[HM + i] = As[buf][kk][BM / 2 + ty * HM + i];
      }
#pragma unroll
      for (int j = 0; j < HN; ++j) {
        b[j] = Bs[buf][kk][tx * HN + j];
        b[HN + j] = Bs[buf][kk][BN / 2 + tx * HN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
    }
    if (kt + 1 < ktiles) {
      store_tiles(buf ^ 1);
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = row0 + ((i < HM) ? ty * HM + i : BM / 2 + ty * HM + (i - HM));
    if (r >= M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c0 = col0 + (h ? BN / 2 : 0) + tx * HN;
      T* dst = C + static_cast<long long>(r) * ldc + c0;
      if (c_vec && HN == V && c0 + HN <= N) {
        Vec v;
        T* e = reinterpret_cast<T*>(&v);
#pragma unroll
        for (int j = 0; j < HN; ++j) e[j] = acc[i][h * HN + j];
        *reinterpret_cast<Vec*>(dst) = v;
      } else {
#pragma unroll
        for (int j = 0; j < HN; ++j)
          if (c0 + j < N) dst[j] = acc[i][h * HN + j];
      }
    }
  }
}

// Tile shapes: the large one for the evaluation's batched scores, the small one
// for the fit, whose products have at most 64 rows.
template <typename T> struct GemmTile;
template <> struct GemmTile<float> {
  static constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8;
  static constexpr bool MMA = false;
};
template <> struct GemmTile<double> {     // FP64 tensor cores, 16 warps of 32x32
  static constexpr int BM = 128, BN = 128, BK = 8, TM = 8, TN = 4;
  static constexpr bool MMA = true;
};
template <typename T> struct SmallGemmTile;
template <> struct SmallGemmTile<float> {
  static constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
  static constexpr bool MMA = false;
};
template <> struct SmallGemmTile<double> {  // 8 warps of 32x32
  static constexpr int BM = 64, BN = 128, BK = 8, TM = 8, TN = 4;
  static constexpr bool MMA = true;
};
// The FMA form for doubles (kept for comparisons and as the check of the tensor-core form).
struct FmaGemmTileDouble {
  static constexpr int BM = 64, BN = 64, BK = 8, TM = 4, TN = 4;
  static constexpr bool MMA = false;
};

// Optional extras of a launch: row gather lists for the operands whose
// contraction index is contiguous, and a split of the contraction index into
// `slices` partial products stored c_slice_stride elements apart.
struct GemmExtras {
  const int64_t* a_gather = nullptr;
  const int64_t* b_gather = nullptr;
  int slices = 1;
  long long c_slice_stride = 0;
  // B with the contraction index as its row index only: rows k with
  // k_owner[k] == skip_owner are left out of the product (and not read)
  const int* k_owner = nullptr;
  int skip_owner = -1;
};

// Tile choice for doubles (tests only, sdcab_test_set "gemm_f64_tile"): 0 = by shape,
// 1 = the block tile of gemm_kernel, 2 / 3 = the pipelined 104-column tile with 64 / 128 rows.
int gemm_f64_tile_mode();
void set_gemm_f64_tile_mode(int mode);

}  // namespace sdcab

#include "gemm_f64_pipe.cuh"

namespace sdcab {

template <typename T, typename G>
int launch_gemm_tile(const T* A, const T* B, T* C, int M, int N, int K, long long lda,
                     long long ldb, long long ldc, bool b_kmajor, cudaStream_t stream,
                     const GemmExtras& x) {
  constexpr int V = 16 / sizeof(T);
  if constexpr (std::is_same<T, double>::value && G::MMA) {
    // few classes: the 104-column tile wastes a twenty-fifth of the tensor-core work at
    // m = 100 where the 128-column tile wastes a fifth
    const int mode = gemm_f64_tile_mode();
    const bool narrow = (mode == 0) ? (N <= 104 || (N > 128 && (N + 103) / 104 * 104 <= (N + 127) / 128 * 128))
                                    : mode >= 2;
    if (narrow) {
      // 128 rows per block halve the reads of the second operand's tile, which pays when that
      // tile is the wide one (column index contiguous) and the rows fill the GPU at one block
      // per SM: 25.3 against 23.7 TFLOP/s at 50 000 x 100 x 50 000; with the contraction index
      // contiguous in both operands 64 rows and three blocks per SM are faster (27.0 / 25.7)
      // ... unless the 128-row blocks fill the GPU's last wave worse: compare the rows the
      // busiest SM works through (ncu: 160 such blocks on 148 SMs ran at 44 % of elapsed cycles
      // with the FP64 tensor pipe active, 81 % while an SM had a block)
      DeviceInfo info;
      const int sms = (get_device_info(&info) == SDCAB_OK && info.sm_count > 0) ? info.sm_count : 148;
      const long long load_tall = ((M + 127) / 128 + sms - 1) / sms * 128LL;
      const long long load_short = ((M + 63) / 64 + sms - 1) / sms * 64LL;
      const bool tall = (mode == 0) ? (!b_kmajor && 100 * load_tall <= 107 * load_short) : mode == 3;
      if (tall) return f64pipe::launch<128, 13>(A, B, C, M, N, K, lda, ldb, ldc, b_kmajor, stream, x);
      return f64pipe::launch<64, 13>(A, B, C, M, N, K, lda, ldb, ldc, b_kmajor, stream, x);
    }
  }
  auto aligned = [&](const void* p, long long ld) {
    return ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && ld % V == 0) ? 1 : 0;
  };
  // slices start at multiples of the tile depth, which keeps 16-byte loads aligned
  int k_per_slice = (K + x.slices - 1) / x.slices;
  k_per_slice = (k_per_slice + G::BK - 1) / G::BK * G::BK;
  if (k_per_slice <= 0) k_per_slice = G::BK;
  const int a_vec = aligned(A, lda), c_vec = aligned(C, ldc) && (x.c_slice_stride % V == 0);
  const int b_vec = aligned(B, ldb);
  dim3 grid((N + G::BN - 1) / G::BN, (M + G::BM - 1) / G::BM, x.slices);
  const int threads = (G::BM / G::TM) * (G::BN / G::TN);
  if (b_kmajor)
    gemm_kernel<T, G::BM, G::BN, G::BK, G::TM, G::TN, true, G::MMA><<<grid, threads, 0, stream>>>(
        A, B, C, M, N, K, lda, ldb, ldc, a_vec, b_vec, c_vec, x.a_gather, x.b_gather, k_per_slice,
        x.c_slice_stride, nullptr, -1);
  else
    gemm_kernel<T, G::BM, G::BN, G::BK, G::TM, G::TN, false, G::MMA><<<grid, threads, 0, stream>>>(
        A, B, C, M, N, K, lda, ldb, ldc, a_vec, b_vec, c_vec, x.a_gather, nullptr, k_per_slice,
        x.c_slice_stride, x.k_owner, x.skip_owner);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

template <typename T>
int launch_gemm(const T* A, const T* B, T* C, int M, int N, int K, long long lda, long long ldb,
                long long ldc, bool b_kmajor, cudaStream_t stream) {
  // doubles: 64-row tiles keep two thread blocks per SM and even out the last wave
  if (sizeof(T) == 8)
    return launch_gemm_tile<T, SmallGemmTile<T>>(A, B, C, M, N, K, lda, ldb, ldc, b_kmajor, stream,
                                                 GemmExtras());
  return launch_gemm_tile<T, GemmTile<T>>(A, B, C, M, N, K, lda, ldb, ldc, b_kmajor, stream,
                                          GemmExtras());
}

}  // namespace sdcab
