// Score GEMM on the fifth-generation tensor cores (sm_100a), paired-CTA form:
// C = A * B' for float operands whose contraction index is contiguous
// (scores = X' W), float accuracy from three TF32 products ("3xTF32").
//
// What bounds a 3xTF32 kernel on this GPU is shared-memory bandwidth, not the
// tensor pipe: the operands of every tcgen05.mma are read from shared memory,
// and the split of each tile into its TF32 head and the remainder reads and
// writes shared memory again.  With 128 x 128 tiles in one CTA a stage moves
// about 230 KB through shared memory for 770 clocks of tensor work at 128 B per
// clock: the pipe was busy 44 % of the time.  This kernel is shaped to move fewer
// bytes per flop:
//
//   * Two CTAs of a cluster (one SM pair) work on one 256 x 256 tile with
//     tcgen05.mma.cta_group::2: each CTA holds 128 rows of A and 128 rows of B
//     per stage and accumulates its 128 x 256 half in its own tensor memory; the
//     B rows are read once per SM and serve both tensor cores.  Each CTA loads
//     its own halves with plain TMA loads (no multicast).
//   * The tensor core truncates its 32-bit operands to TF32 by itself, so the tile
//     as TMA delivered it serves as the head term; the worker warps only write the
//     remainder  lo = x - tf32(x)  (exact in float) to a second buffer.  A build
//     switch keeps the explicit head (hi written in place) for comparison.
//   * Raw tiles and remainder tiles live in rings of their own (4 and 3 deep):
//     TMA runs up to four stages ahead of the tensor core, the split up to two.
//   * The kernel is persistent: a pair walks over the tiles t = pair, pair + P, ...
//     with the class tile as the fast index, so that the pairs working at the same
//     time share their rows of X through L2.
//   * The tensor core adds into its accumulator with truncation, which shows after
//     a few hundred additions; the contraction is cut into chunks of kChunk stages
//     that alternate between two TMEM accumulators, and the worker warps drain each
//     finished chunk into float registers (rounded additions) while the next chunk
//     is being multiplied, across tile boundaries.
//
// The same kernel serves the product with the contraction index as the SLOW index of
// both operands (template flag kMN): W = A' X, primal variables from dual variables
// (include/sdca/solver/eval/core.h:164-174 of the reference), where example i holds m
// contiguous dual variables and d contiguous features.  The operand tiles are then
// "MN-major": TMA brings boxes of 32 contiguous floats x 32 examples, a stage is four such
// boxes per operand (written with the 32-byte-atom form of the 128-byte swizzle, the
// only MN-major layout the tensor core takes for 32-bit operands), the shared-memory
// descriptors name the stride between the boxes, and one MMA consumes a group of 8
// examples (1024 bytes further per step).  The split into
// head and remainder is elementwise, so it does not care.
//
// Roles per CTA (12 warps): warp 0 lane 0 issues TMA; warp 1 owns tensor memory
// and, in the leader CTA (cluster rank 0), lane 0 issues every tcgen05.mma of the
// pair; warps 2-3 only give up their registers; warps 4-11 split and drain.  Hand-overs go through mbarriers; the workers
// of both CTAs arrive on the leader's barriers through the cluster's shared
// address space, the tensor core's completions are multicast to both CTAs.
// Every wait is bounded: a wait that runs out raises an error word in global
// memory that the host returns as a status; all roles then leave their loops, the
// cluster synchronises, tensor memory is freed and the kernel ends.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common_host.h"
#include "gemm_tc.cuh"   // TMA descriptor encoding, mbarrier and descriptor helpers

namespace sdcab {
namespace tc2 {

constexpr int kBM = 128;          // rows of A per CTA (256 per pair)
constexpr int kBNHalf = 128;      // rows of B per CTA
constexpr int kBN = 256;          // columns of the pair's tile = accumulator columns per CTA
constexpr int kBK = 32;           // floats per row of a stage = one 128-byte swizzle row
constexpr int kRawStages = 4;
constexpr int kLoStages = 3;
constexpr int kChunk = 4;         // stages per TMEM accumulation chunk (128 contraction steps)
constexpr int kWorkerWarps = 8;
constexpr int kControlWarps = 4;  // one warpgroup: TMA, MMA + tensor memory, two idle warps
constexpr int kThreads = 32 * (kControlWarps + kWorkerWarps);
// Every quarter of the SM's register file hosts one control warp and two worker warps.
// A worker keeps 128 running sums in registers, so the control warpgroup hands most of
// its registers over (setmaxnreg).  The pool is what the launch allocated: the kernel's
// register count (168 for 384 threads) times 384 = 64512.  setmaxnreg.inc blocks until
// its registers are there, for ever if the numbers do not add up, so they are checked at
// compile time against 168 and at run time against the count the compiler really chose:
// 80 * 128 + 208 * 256 = 63488 <= 64512.  (The thread that issues the MMAs needs its
// descriptors and barrier addresses in registers: with 56 it spilled inside the issue
// loop, which is the critical path of the whole pair.)
constexpr int kControlRegs = 80;
constexpr int kWorkerRegs = 208;
constexpr int kPoolRegsNeeded = kControlRegs * 32 * kControlWarps + kWorkerRegs * 32 * kWorkerWarps;
static_assert(kPoolRegsNeeded <= 168 * kThreads, "setmaxnreg would wait for registers that never come");
constexpr int kTileBytes = kBM * kBK * 4;                     // 16 KB, A and B halves alike
constexpr int kRawBytes = 2 * kTileBytes;                     // A then B
constexpr int kBoxBytes = 32 * kBK * 4;                       // MN-major: 32 floats x 32 examples
constexpr int kSmemTiles = kRawStages * kRawBytes + kLoStages * kRawBytes;
constexpr int kNumBarriers = 2 * kRawStages + 2 * kLoStages + 5;
static_assert(kNumBarriers * 8 <= 256, "barrier area");
constexpr int kSmemBytes = kSmemTiles + 1024 /* alignment */ + 256 /* barriers */;
constexpr unsigned kSpinLimit = 1u << 22;
constexpr unsigned kSpinLimitShort = 1u << 11;

using tc::mbar_init;
using tc::mbar_expect_tx;
using tc::smem_desc_sw128;
using tc::smem_u32;
using tc::tma_load_2d;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  // Default semantics (release at CTA scope) on purpose: what the arrival publishes is
  // shared memory of the arriving CTA, already ordered for the tensor core by
  // fence.proxy.async, or a finished tcgen05.ld.  The cluster-scope release form cost
  // about a thousand clocks per stage here (3.2 ms -> 2.3 ms for 65 536 examples).
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait on a barrier of this CTA (arrivals may come from the peer CTA):
// false, with the error word set, when the limit is reached or somebody else has
// already failed.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, int* err, int code,
                                         unsigned limit) {
  for (unsigned i = 0; i < limit; ++i) {
    if (mbar_try_cluster(bar, parity)) return true;
    if (i > 2048) __nanosleep(64);
    if ((i & 255) == 255 && *reinterpret_cast<volatile int*>(err) != 0) return false;
  }
  atomicCAS(err, 0, code);
  return false;
}

// D (float, TMEM of both CTAs) += A (TF32, smem) * B (TF32, smem), 256 x 256 x 8 per pair
__device__ __forceinline__ void mma_tf32_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on the barrier at this offset in both CTAs once all MMAs issued so far are done
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask) : "memory");
}

// MN-major operand.  For 32-bit operands the tensor core takes MN-major tiles in one
// layout only, the 128-byte swizzle with 32-byte atoms: rows of 32 contiguous floats
// along M (or N), 4 rows (contraction steps) per 512-byte swizzle atom, the 32-byte
// pieces of a row exchanged among themselves by the row's index (TMA's
// SWIZZLE_128B_ATOM_32B writes exactly this).  The next 32 floats along M / N lie
// `box_bytes` further (leading byte offset), the next 4 contraction steps 512 bytes
// further (stride byte offset); descriptor version 1, layout type 1.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t box_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((box_bytes >> 4) & 0x3FFF) << 16;   // leading byte offset
  d |= static_cast<uint64_t>(512 >> 4) << 32;                    // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                           // version
  d |= static_cast<uint64_t>(1) << 61;                           // SWIZZLE_128B_BASE32B
  return d;
}

struct Params {
  float* C;
  const float* C0;           // optional addend with the layout of C (W0), or null
  long long ldc;
  int M, N, K;
  int tiles_m, tiles_n;      // 256 x 256 tiles
  int* err;
  unsigned spin_limit;
  int lose_tile;             // test switch: the leader's TMA skips this stage (-1: none)
};

template <bool kWriteHi, bool kMN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                        const __grid_constant__ CUtensorMap map_b, Params p) {
  extern __shared__ unsigned char smem_dyn[];
  // 1024-byte alignment: the swizzle pattern is a function of address bits 7-9
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
  unsigned char* raw_base = smem;
  unsigned char* lo_base = smem + kRawStages * kRawBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles);
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int ktiles = (p.K + kBK - 1) / kBK;
  const int chunks_per_tile = (ktiles + kChunk - 1) / kChunk;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int my_tiles = (pair < num_tiles) ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
  const unsigned limit = p.spin_limit;

  // barriers: raw tile landed / raw stage free / lo written (counted in the leader) /
  // lo stage free / accumulator holds a finished chunk / accumulator drained (leader)
  auto bar_full = [&](int s) { return smem_u32(&bars[s]); };
  auto bar_raw_free = [&](int s) { return smem_u32(&bars[kRawStages + s]); };
  auto bar_ready = [&](int s) { return smem_u32(&bars[2 * kRawStages + s]); };
  auto bar_lo_free = [&](int s) { return smem_u32(&bars[2 * kRawStages + kLoStages + s]); };
  auto bar_acc_full = [&](int b) { return smem_u32(&bars[2 * kRawStages + 2 * kLoStages + b]); };
  auto bar_acc_free = [&](int b) { return smem_u32(&bars[2 * kRawStages + 2 * kLoStages + 2 + b]); };
  auto bar_done = [&]() { return smem_u32(&bars[2 * kRawStages + 2 * kLoStages + 4]); };
  auto a_raw = [&](int s) { return raw_base + s * kRawBytes; };
  auto b_raw = [&](int s) { return raw_base + s * kRawBytes + kTileBytes; };
  auto a_lo = [&](int s) { return lo_base + s * kRawBytes; };
  auto b_lo = [&](int s) { return lo_base + s * kRawBytes + kTileBytes; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_raw_free(s), 1); }
    for (int s = 0; s < kLoStages; ++s) {
      mbar_init(bar_ready(s), 2 * kWorkerWarps);   // the worker warps of both CTAs
      mbar_init(bar_lo_free(s), 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full(b), 1); mbar_init(bar_acc_free(b), 2 * kWorkerWarps); }
    mbar_init(bar_done(), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"(static_cast<uint32_t>(2 * kBN)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  // both CTAs must have their barriers initialised before anybody signals across
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_slot;

  if (warp < kControlWarps) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kControlRegs));
  if (warp == 0) {
    // ---- TMA producer: this CTA's 128 rows of A and 128 rows of B per stage ------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      int last_issue[kRawStages];
#pragma unroll
      for (int s = 0; s < kRawStages; ++s) last_issue[s] = -1;
      for (int ti = 0; ti < my_tiles && ok; ++ti) {
        const int t = pair + ti * num_pairs;
        const int m0 = (t / p.tiles_n) * (2 * kBM) + static_cast<int>(rank) * kBM;
        const int n0 = (t % p.tiles_n) * kBN + static_cast<int>(rank) * kBNHalf;
        for (int kt = 0; kt < ktiles; ++kt, ++it) {
          const int s = it % kRawStages;
          ok = wait_bar(bar_raw_free(s), ((it / kRawStages) & 1) ^ 1, p.err, 1, limit);
          if (!ok) break;
          if (it == p.lose_tile && rank == 0) continue;   // test switch: this stage never lands
          mbar_expect_tx(bar_full(s), kRawBytes);
          if (kMN) {
            // four boxes of 32 floats x 32 examples per operand
#pragma unroll
            for (int c = 0; c < kBM / 32; ++c) {
              tma_load_2d(smem_u32(a_raw(s)) + c * kBoxBytes, &map_a, m0 + 32 * c, kt * kBK, bar_full(s));
              tma_load_2d(smem_u32(b_raw(s)) + c * kBoxBytes, &map_b, n0 + 32 * c, kt * kBK, bar_full(s));
            }
          } else {
            tma_load_2d(smem_u32(a_raw(s)), &map_a, kt * kBK, m0, bar_full(s));
            tma_load_2d(smem_u32(b_raw(s)), &map_b, kt * kBK, n0, bar_full(s));
          }
#pragma unroll
          for (int q = 0; q < kRawStages; ++q) if (q == s) last_issue[q] = it;
        }
      }
      // Copies still in flight must have landed before this CTA's shared memory is given
      // up; when everything went well the workers have seen them all and this costs nothing.
#pragma unroll
      for (int s = 0; s < kRawStages; ++s)
        if (last_issue[s] >= 0)
          wait_bar(bar_full(s), (last_issue[s] / kRawStages) & 1, p.err, 8, limit);
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one thread of the leader CTA drives both tensor cores --------
    if (lane == 0 && rank == 0) {
      // instruction descriptor: D = F32, A = B = TF32, both K-major, N = 256, M = 256 (pair)
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) |
                             (kMN ? ((1u << 15) | (1u << 16)) : 0u) |      // both operands MN-major
                             (static_cast<uint32_t>(kBN >> 3) << 17) |
                             (static_cast<uint32_t>((2 * kBM) >> 4) << 24);
      int it = 0, ch = 0;
      bool ok = true;
      for (int ti = 0; ti < my_tiles && ok; ++ti) {
        for (int kt = 0; kt < ktiles && ok; ++kt, ++it) {
          const int s4 = it % kRawStages, s2 = it % kLoStages;
          const bool chunk_first = (kt % kChunk) == 0;
          const bool chunk_last = (kt % kChunk) == kChunk - 1 || kt == ktiles - 1;
          const int b = ch & 1;
          if (chunk_first) {
            // accumulator b must have been drained of the chunk that used it before
            ok = wait_bar(bar_acc_free(b), ((ch >> 1) & 1) ^ 1, p.err, 6, limit);
            if (!ok) break;
          }
          // the workers arrive after they have seen the raw tile and written lo
          ok = wait_bar(bar_ready(s2), (it / kLoStages) & 1, p.err, 3, limit);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(b * kBN);
          const uint64_t da_hi = kMN ? smem_desc_mn_sw128(smem_u32(a_raw(s4)), kBoxBytes) : smem_desc_sw128(smem_u32(a_raw(s4)));
          const uint64_t db_hi = kMN ? smem_desc_mn_sw128(smem_u32(b_raw(s4)), kBoxBytes) : smem_desc_sw128(smem_u32(b_raw(s4)));
          const uint64_t da_lo = kMN ? smem_desc_mn_sw128(smem_u32(a_lo(s2)), kBoxBytes) : smem_desc_sw128(smem_u32(a_lo(s2)));
          const uint64_t db_lo = kMN ? smem_desc_mn_sw128(smem_u32(b_lo(s2)), kBoxBytes) : smem_desc_sw128(smem_u32(b_lo(s2)));
#pragma unroll
          for (int ks = 0; ks < kBK / 8; ++ks) {
            // one MMA takes 8 contraction steps: 32 bytes along a K-major row, or the next
            // group of 8 rows (1024 bytes) of an MN-major box
            const uint64_t off = static_cast<uint64_t>((kMN ? ks * 1024 : ks * 32) >> 4);
            // small terms first, the large product last
            mma_tf32_pair(tmem_d, da_lo + off, db_hi + off, idesc, !(chunk_first && ks == 0));
            mma_tf32_pair(tmem_d, da_hi + off, db_lo + off, idesc, 1);
            mma_tf32_pair(tmem_d, da_hi + off, db_hi + off, idesc, 1);
          }
          mma_commit_pair(bar_raw_free(s4));
          mma_commit_pair(bar_lo_free(s2));
          if (chunk_last) { mma_commit_pair(bar_acc_full(b)); ++ch; }
        }
      }
      // whatever was issued has to be finished before tensor memory is freed, also when a
      // wait ran out somewhere and the roles are leaving early
      if (it > 0) {
        mma_commit_pair(bar_done());
        wait_bar(bar_done(), 0, p.err, 9, limit);
      }
    }
  }
  } else {
    // ---- workers (warps 4..11): split every stage, drain finished chunks, store ---
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kWorkerRegs));
    const int wt = threadIdx.x - 32 * kControlWarps;   // 0..255
    const int quarter = warp & 3;               // TMEM lanes 32*quarter .. +31 belong to this warp
    const int half = (warp - kControlWarps) >> 2;      // accumulator columns 128*half .. +127
    uint32_t ready_remote[kLoStages];
#pragma unroll
    for (int s = 0; s < kLoStages; ++s) ready_remote[s] = map_to_rank(bar_ready(s), 0);
    const uint32_t acc_free_remote[2] = {map_to_rank(bar_acc_free(0), 0), map_to_rank(bar_acc_free(1), 0)};
    float acc[kBN / 2];
#pragma unroll
    for (int j = 0; j < kBN / 2; ++j) acc[j] = 0.0f;
    bool ok = true;
    const int total_chunks = my_tiles * chunks_per_tile;
    int drained = 0;                            // chunks drained so far (over all tiles)

    // adds chunk `c` (global index) from its TMEM accumulator into acc; after the last
    // chunk of a tile the tile is stored
    auto drain = [&](int c) -> bool {
      const int b = c & 1;
      const bool first = (c % chunks_per_tile) == 0;
      if (!wait_bar(bar_acc_full(b), (c >> 1) & 1, p.err, 5, limit)) return false;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
      for (int c0 = 0; c0 < kBN / 2; c0 += 16) {
        // 16 columns at a time: the 128 running sums leave few registers for temporaries
        uint32_t r[16];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               static_cast<uint32_t>(b * kBN + half * (kBN / 2) + c0);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
              "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
              "=r"(r[14]), "=r"(r[15])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        // the first chunk of a tile starts the sums anew (here, not by a reset of the
        // registers after the store: that makes the compiler keep a second copy of the 128
        // sums); `first` is the same for the whole warp
        if (first) {
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c0 + j] = __uint_as_float(r[j]);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[c0 + j] += __uint_as_float(r[j]);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc_free_remote[b]);
      if (c % chunks_per_tile == chunks_per_tile - 1) {
        const int t = pair + (c / chunks_per_tile) * num_pairs;
        const int row = (t / p.tiles_n) * (2 * kBM) + static_cast<int>(rank) * kBM + quarter * 32 + lane;
        const int col0 = (t % p.tiles_n) * kBN + half * (kBN / 2);
        const bool vec_ok = ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
        if (row < p.M) {
          float* dst = p.C + static_cast<long long>(row) * p.ldc + col0;
          const float* add = p.C0 ? p.C0 + static_cast<long long>(row) * p.ldc + col0 : nullptr;
          if (vec_ok && col0 + kBN / 2 <= p.N && (!add || (reinterpret_cast<uintptr_t>(p.C0) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < kBN / 2; j += 4) {
              float4 o = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
              if (add) {
                const float4 w0 = *reinterpret_cast<const float4*>(add + j);
                o.x += w0.x; o.y += w0.y; o.z += w0.z; o.w += w0.w;
              }
              *reinterpret_cast<float4*>(dst + j) = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < kBN / 2; ++j)
              if (col0 + j < p.N) dst[j] = add ? acc[j] + add[j] : acc[j];
          }
        }
      }
      return true;
    };
    // last stage (global index) of chunk c
    auto chunk_end = [&](int c) {
      const int ti = c / chunks_per_tile, cc = c % chunks_per_tile;
      const int last = (cc + 1) * kChunk - 1;
      return ti * ktiles + (last < ktiles - 1 ? last : ktiles - 1);
    };

    const int total_stages = my_tiles * ktiles;
    // one loop, one call site of the drain: stages are split while there are any, and the
    // iterations after the last stage only drain what is left
    for (int it = 0; ok && (it < total_stages || drained < total_chunks); ++it) {
      if (it < total_stages) {
        const int s4 = it % kRawStages, s2 = it % kLoStages;
        ok = wait_bar(bar_full(s4), (it / kRawStages) & 1, p.err, 4, limit) &&
             wait_bar(bar_lo_free(s2), ((it / kLoStages) & 1) ^ 1, p.err, 7, limit);
        if (!ok) break;
        float4* ar = reinterpret_cast<float4*>(a_raw(s4));   // A then B, contiguous
        float4* al = reinterpret_cast<float4*>(a_lo(s2));
#pragma unroll
        for (int j = 0; j < kRawBytes / 16 / (32 * kWorkerWarps); ++j) {
          const int i = wt + j * 32 * kWorkerWarps;
          const float4 v = ar[i];
          float4 h, l;
          h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u); l.x = v.x - h.x;
          h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u); l.y = v.y - h.y;
          h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u); l.z = v.z - h.z;
          h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u); l.w = v.w - h.w;
          if (kWriteHi) ar[i] = h;
          al[i] = l;
        }
        // generic-proxy writes must be visible to the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int q = 0; q < kLoStages; ++q) if (q == s2) mbar_arrive_cluster(ready_remote[q]);
        }
      }
      // A chunk whose last stage was split kLoStages stages ago has been multiplied: the
      // split just done had to wait for that stage's lo buffer, which the tensor core
      // releases together with the chunk.
      if (drained < total_chunks && (it >= total_stages || it >= chunk_end(drained) + kLoStages)) {
        ok = drain(drained);
        ++drained;
      }
    }
  }

  // nobody leaves, and tensor memory stays allocated, until both CTAs are done: the
  // leader's tensor-core work reads the peer's shared memory and writes its tensor memory
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"(static_cast<uint32_t>(2 * kBN)) : "memory");
  }
}

// Whether the paired kernel can take this problem (alignment rules of TMA).
inline bool usable(const float* A, const float* B, long long lda, long long ldb) {
  return tc::usable(A, B, lda, ldb);
}

// C (M x N, ldc) = A (M x K, lda) * B' (B is N x K, ldb).  err_dev: one int in
// device memory, zero on entry; non-zero afterwards means a wait ran out.
inline int launch(const float* A, const float* B, float* C, int M, int N, int K, long long lda,
                  long long ldb, long long ldc, int* err_dev, bool write_hi, bool lose_a_tile,
                  cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  if (!tc::make_map(&map_a, A, M, K, lda, kBM) || !tc::make_map(&map_b, B, N, K, ldb, kBNHalf))
    return SDCAB_ERR_CUDA;
  auto kernel = write_hi ? gemm_tf32x3_pair_kernel<true, false> : gemm_tf32x3_pair_kernel<false, false>;
  // the opt-in to large dynamic shared memory is a property of the function on each
  // device, so it is set on every launch (a cheap host-side call)
  SDCAB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;
  // the register hand-over inside the kernel needs the pool it was sized for
  cudaFuncAttributes attr;
  SDCAB_CUDA_TRY(cudaFuncGetAttributes(&attr, kernel));
  if (attr.numRegs * kThreads < kPoolRegsNeeded) return SDCAB_ERR_NOT_IMPLEMENTED;
  Params p;
  p.C = C; p.C0 = nullptr; p.ldc = ldc; p.M = M; p.N = N; p.K = K; p.err = err_dev;
  p.tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
  p.tiles_n = (N + kBN - 1) / kBN;
  p.spin_limit = lose_a_tile ? kSpinLimitShort : kSpinLimit;
  p.lose_tile = lose_a_tile ? 1 : -1;
  // one pair of CTAs per pair of SMs, or fewer when there are fewer tiles
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  int pairs = std::max(1, info.sm_count / 2);
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  kernel<<<2 * pairs, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

// box = 32 contiguous floats x 32 rows of a rows x cols matrix (row stride ld floats)
inline bool make_map_mn(CUtensorMap* map, const float* base, long long rows, long long cols, long long ld) {
  tc::EncodeTiledFn fn = tc::encode_tiled();
  if (!fn) return false;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * sizeof(float)};
  cuuint32_t box[2] = {32, static_cast<cuuint32_t>(kBK)};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Whether the MN-major form can take C = A' B (+ C0): TMA's alignment rules.
inline bool usable_mn(const float* A, const float* B, const float* C0, long long lda, long long ldb) {
  return ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) == 0 &&
         (lda % 4) == 0 && (ldb % 4) == 0 && tc::encode_tiled() != nullptr &&
         (!C0 || (reinterpret_cast<uintptr_t>(C0) & 3) == 0);
}

// C (M x N, ldc) = A' B [+ C0] with A: K x M (row stride lda), B: K x N (row stride ldb):
// the contraction index is the slow index of both operands.  err_dev as in launch().
inline int launch_mn(const float* A, const float* B, const float* C0, float* C, int M, int N, long long K,
                     long long lda, long long ldb, long long ldc, int* err_dev, cudaStream_t stream) {
  if (K > 0x7fffffffLL - kBK) return SDCAB_ERR_TOO_LARGE;
  CUtensorMap map_a, map_b;
  if (!make_map_mn(&map_a, A, K, M, lda) || !make_map_mn(&map_b, B, K, N, ldb)) return SDCAB_ERR_CUDA;
  auto kernel = gemm_tf32x3_pair_kernel<false, true>;
  SDCAB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;
  cudaFuncAttributes attr;
  SDCAB_CUDA_TRY(cudaFuncGetAttributes(&attr, kernel));
  if (attr.numRegs * kThreads < kPoolRegsNeeded) return SDCAB_ERR_NOT_IMPLEMENTED;
  Params p;
  p.C = C; p.C0 = C0; p.ldc = ldc; p.M = M; p.N = N; p.K = static_cast<int>(K); p.err = err_dev;
  p.tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
  p.tiles_n = (N + kBN - 1) / kBN;
  p.spin_limit = kSpinLimit;
  p.lose_tile = -1;
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  int pairs = std::max(1, info.sm_count / 2);
  if (tiles < pairs) pairs = static_cast<int>(tiles);
  kernel<<<2 * pairs, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

}  // namespace tc2
}  // namespace sdcab
