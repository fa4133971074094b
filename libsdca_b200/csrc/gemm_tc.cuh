// Score GEMM on the fifth-generation tensor cores (sm_100a): C = A * B' for
// float operands whose contraction index is contiguous (scores = X' W).
//
//   * TMA (cp.async.bulk.tensor, 128-byte swizzle) brings 128 x 32 float tiles
//     of A and B into shared memory; no thread touches global memory for loads.
//   * Four worker warps split every tile in place into hi = the value with the
//     13 low mantissa bits cleared (exactly a TF32 number) and lo = x - hi
//     (exact in float), so that  a*b ~= hi*hi + hi*lo + lo*hi  recovers float
//     accuracy from TF32 products ("3xTF32"); the dropped lo*lo term is 2^-22
//     relative.  The split is elementwise, so it works on the swizzled bytes.
//   * One elected thread issues tcgen05.mma (kind::tf32, 128 x 128 x 8 per
//     instruction, cta_group::1) on shared-memory descriptors; the 128 x 128
//     float accumulator lives in tensor memory (128 TMEM columns).
//   * The tensor core adds into its accumulator with truncation, which shows
//     after a few hundred additions; so the contraction is cut into chunks of
//     kChunk tiles that alternate between two TMEM accumulators, and the worker
//     warps drain each finished chunk with tcgen05.ld into float registers
//     (rounded additions) while the next chunk is being multiplied.  At the end
//     they store the scores from those registers.
// Stages are handed over through mbarriers.  Every wait is bounded: a wait that
// runs out raises an error word that the host returns as a status; the kernel
// then drains, frees its tensor memory and exits.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common_host.h"

namespace sdcab {
namespace tc {

constexpr int kBM = 128;        // rows of A per tile (examples)
constexpr int kBN = 128;        // rows of B per tile (classes) = TMEM columns
constexpr int kBK = 32;         // floats per row of a tile = one 128-byte swizzle row
constexpr int kStages = 3;
constexpr int kChunk = 4;        // k-tiles per TMEM accumulation chunk (128 contraction steps)
constexpr int kDrainLag = 2;     // tiles the drain of a chunk trails its last split
constexpr int kThreads = 192;   // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: split + epilogue
constexpr int kTileBytesA = kBM * kBK * 4;
constexpr int kTileBytesB = kBN * kBK * 4;
constexpr int kStageBytes = 2 * kTileBytesA + 2 * kTileBytesB;   // raw/hi and lo of both
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment */ + 256 /* barriers */;
constexpr unsigned kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false (and the error word set) when the limit is reached or
// another role has already failed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err, int code) {
  for (unsigned i = 0; i < kSpinLimit; ++i) {
    if (mbar_try(bar, parity)) return true;
    if (i > 64) __nanosleep(32);
    if ((i & 1023) == 1023 && *reinterpret_cast<volatile int*>(err) != 0) return false;
  }
  atomicCAS(err, 0, code);
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}

// K-major operand, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024
// bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>(1) << 16;            // leading byte offset (unused with swizzle): 1
  d |= static_cast<uint64_t>(1024 >> 4) << 32;    // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;            // version
  d |= static_cast<uint64_t>(2) << 61;            // SWIZZLE_128B
  return d;
}

// D (float, TMEM) += A (TF32, smem, K-major) * B (TF32, smem, K-major)
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar) : "memory");
}

struct Params {
  float* C;
  long long ldc;
  int M, N, K;
  int* err;
};

// (internal linkage: the header is included by more than one translation unit)
static __global__ void __launch_bounds__(kThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a,
                   const __grid_constant__ CUtensorMap map_b, Params p) {
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment: the swizzle pattern is a function of address bits 7-9
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  // bars[0..S): raw tiles landed, [S..2S): lo tiles written, [2S..3S): stage free,
  // [3S], [3S+1]: accumulator b holds a finished chunk, [3S+2], [3S+3]: accumulator b drained
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
  const int ktiles = (p.K + kBK - 1) / kBK;

  auto bar_full = [&](int s) { return smem_u32(&bars[s]); };
  auto bar_lo = [&](int s) { return smem_u32(&bars[kStages + s]); };
  auto bar_free = [&](int s) { return smem_u32(&bars[2 * kStages + s]); };
  auto bar_acc_full = [&](int b) { return smem_u32(&bars[3 * kStages + b]); };
  auto bar_acc_free = [&](int b) { return smem_u32(&bars[3 * kStages + 2 + b]); };
  auto a_raw = [&](int s) { return smem + s * kStageBytes; };
  auto a_lo = [&](int s) { return smem + s * kStageBytes + kTileBytesA; };
  auto b_raw = [&](int s) { return smem + s * kStageBytes + 2 * kTileBytesA; };
  auto b_lo = [&](int s) { return smem + s * kStageBytes + 2 * kTileBytesA + kTileBytesB; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_lo(s), 4);
      mbar_init(bar_free(s), 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full(b), 1); mbar_init(bar_acc_free(b), 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(static_cast<uint32_t>(2 * kBN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------
    if (lane == 0) {
      for (int kt = 0; kt < ktiles; ++kt) {
        const int s = kt % kStages;
        const uint32_t parity = ((kt / kStages) & 1) ^ 1;
        if (!mbar_wait(bar_free(s), parity, p.err, 1)) break;
        mbar_expect_tx(bar_full(s), kTileBytesA + kTileBytesB);
        tma_load_2d(smem_u32(a_raw(s)), &map_a, kt * kBK, m0, bar_full(s));
        tma_load_2d(smem_u32(b_raw(s)), &map_b, kt * kBK, n0, bar_full(s));
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------
    if (lane == 0) {
      // instruction descriptor: D = F32, A = B = TF32, both K-major, N = 128, M = 128
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) |
                             (static_cast<uint32_t>(kBN >> 3) << 17) |
                             (static_cast<uint32_t>(kBM >> 4) << 24);
      bool ok = true;
      for (int kt = 0; kt < ktiles && ok; ++kt) {
        const int s = kt % kStages;
        const uint32_t parity = (kt / kStages) & 1;
        const int chunk = kt / kChunk, b = chunk & 1;
        const bool chunk_first = (kt % kChunk) == 0;
        if (chunk_first) {
          // accumulator b must have been drained of the chunk that used it before
          ok = mbar_wait(bar_acc_free(b), ((chunk >> 1) & 1) ^ 1, p.err, 6);
          if (!ok) break;
        }
        ok = mbar_wait(bar_full(s), parity, p.err, 2) && mbar_wait(bar_lo(s), parity, p.err, 3);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(b * kBN);
        const uint64_t da_hi = smem_desc_sw128(smem_u32(a_raw(s)));
        const uint64_t da_lo = smem_desc_sw128(smem_u32(a_lo(s)));
        const uint64_t db_hi = smem_desc_sw128(smem_u32(b_raw(s)));
        const uint64_t db_lo = smem_desc_sw128(smem_u32(b_lo(s)));
#pragma unroll
        for (int ks = 0; ks < kBK / 8; ++ks) {
          const uint64_t off = static_cast<uint64_t>(ks * 32 >> 4);  // 8 floats = 32 bytes
          // small terms first, the large product last
          mma_tf32(tmem_d, da_lo + off, db_hi + off, idesc, !(chunk_first && ks == 0));
          mma_tf32(tmem_d, da_hi + off, db_lo + off, idesc, 1);
          mma_tf32(tmem_d, da_hi + off, db_hi + off, idesc, 1);
        }
        mma_commit(bar_free(s));
        if ((kt % kChunk) == kChunk - 1 || kt == ktiles - 1) mma_commit(bar_acc_full(b));
      }
    }
  } else {
    // ---- split workers (warps 2..5), then epilogue ------------------------------
    const int wt = threadIdx.x - 64;  // 0..127
    const int quarter = warp & 3;     // TMEM lanes 32*quarter .. +31 belong to this warp
    const int nchunks = (ktiles + kChunk - 1) / kChunk;
    float acc[kBN];
#pragma unroll
    for (int j = 0; j < kBN; ++j) acc[j] = 0.0f;
    bool ok = true;
    // adds the finished chunk `chunk` from its TMEM accumulator into acc
    auto drain = [&](int chunk) -> bool {
      const int b = chunk & 1;
      if (!mbar_wait(bar_acc_full(b), (chunk >> 1) & 1, p.err, 5)) return false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               static_cast<uint32_t>(b * kBN + c0);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
              "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
              "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
              "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
              "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c0 + j] += __uint_as_float(r[j]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_free(b));
      return true;
    };
    int drained = 0;
    for (int kt = 0; kt < ktiles && ok; ++kt) {
      const int s = kt % kStages;
      const uint32_t parity = (kt / kStages) & 1;
      ok = mbar_wait(bar_full(s), parity, p.err, 4);
      if (!ok) break;
      float4* ar = reinterpret_cast<float4*>(a_raw(s));
      float4* al = reinterpret_cast<float4*>(a_lo(s));
      float4* br = reinterpret_cast<float4*>(b_raw(s));
      float4* bl = reinterpret_cast<float4*>(b_lo(s));
      auto split = [](float x, float& hi, float& lo) {
        hi = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
        lo = x - hi;
      };
#pragma unroll 4
      for (int i = wt; i < kTileBytesA / 16; i += 128) {
        float4 v = ar[i], h, l;
        split(v.x, h.x, l.x); split(v.y, h.y, l.y); split(v.z, h.z, l.z); split(v.w, h.w, l.w);
        ar[i] = h; al[i] = l;
      }
#pragma unroll 4
      for (int i = wt; i < kTileBytesB / 16; i += 128) {
        float4 v = br[i], h, l;
        split(v.x, h.x, l.x); split(v.y, h.y, l.y); split(v.z, h.z, l.z); split(v.w, h.w, l.w);
        br[i] = h; bl[i] = l;
      }
      // generic-proxy writes must be visible to the tensor core (async proxy)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_lo(s));
      // drain the chunk whose last tile was split kDrainLag tiles ago
      const int done_tiles = kt + 1 - kDrainLag;
      if (done_tiles > 0 && done_tiles % kChunk == 0 && drained < done_tiles / kChunk) {
        ok = drain(drained);
        ++drained;
      }
    }
    while (ok && drained < nchunks) { ok = drain(drained); ++drained; }
    if (ok) {
      const int row = m0 + quarter * 32 + lane;
      const bool vec_ok = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
      if (row < p.M) {
        float* dst = p.C + static_cast<long long>(row) * p.ldc + n0;
        if (vec_ok && n0 + kBN <= p.N) {
#pragma unroll
          for (int j = 0; j < kBN; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < kBN; ++j)
            if (n0 + j < p.N) dst[j] = acc[j];
        }
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"(static_cast<uint32_t>(2 * kBN)) : "memory");
  }
}

// ---- host side ----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// rows x K float matrix, row stride ld floats; box = kBK floats x box_rows rows
inline bool make_map(CUtensorMap* map, const float* base, long long rows, long long K,
                     long long ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * sizeof(float)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Whether the tensor-core path can take this problem (alignment rules of TMA).
inline bool usable(const float* A, const float* B, long long lda, long long ldb) {
  return ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 &&
         (lda % 4) == 0 && (ldb % 4) == 0 && encode_tiled() != nullptr;
}

// C (M x N, ldc) = A (M x K, lda) * B' (B is N x K, ldb).  err_dev: one int in
// device memory, zero on entry; non-zero afterwards means a wait ran out.
inline int launch(const float* A, const float* B, float* C, int M, int N, int K, long long lda,
                  long long ldb, long long ldc, int* err_dev, cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  if (!make_map(&map_a, A, M, K, lda, kBM) || !make_map(&map_b, B, N, K, ldb, kBN))
    return SDCAB_ERR_CUDA;
  // the opt-in to large dynamic shared memory is a property of the function on
  // each device, so it is set on every launch (a cheap host-side call)
  SDCAB_CUDA_TRY(cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kSmemBytes));
  Params p;
  p.C = C; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.err = err_dev;
  dim3 grid((N + kBN - 1) / kBN, (M + kBM - 1) / kBM);
  gemm_tf32x3_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

}  // namespace tc
}  // namespace sdcab
