// Loss stage of the evaluation for the top-k hinge objectives on float scores, with
// the score row of an example in registers.
//
// The general loss kernel (eval_loss_kernel) stages every score row in shared memory
// and runs the objective's routines on index-skipping views of it: about 1700 warp
// instructions per example of 1000 scores for the top-k hinge, and for the smooth
// form the general threshold search of the top-k simplex projection over the whole
// row.  Here a warp reads the row with 16-byte loads into registers (eight vectors
// per lane hold 1024 scores), forms  h_j = s_j + (1 - s_y)  in place with the
// label's entry set to -inf, counts the rank on the way, and then
//   gamma = 0  (include/sdca/solver/objective/l2_hinge_topk.h:71-86,
//               l2_topk_hinge.h:72-87): the k largest h by per-lane register buffers
//               and k pops, as topk_sums does on any row;
//   gamma > 0  (l2_hinge_topk.h:162-179): the thresholds of the top-k simplex
//               projection from the candidate path of the batched operator
//               (fast_topk_simplex: lane maxima, cut, compaction, sorted candidates),
//               then <h, p> - 0.5 <p, p> from the thresholds in one pass over the row
//               read a second time from L2.  Rows the candidate path declines take the
//               general routine on a shared-memory copy, like the general kernel.
// Sums, block partials and the rank histogram are those of the general kernel.
//
// Included by eval.cu after LossArgs and the general kernel's constants.
#pragma once

#include "fast_rows.cuh"
#include "losses.cuh"

namespace sdcab {

// h as a row for the routines of losses.cuh: the register row with the label's entry
// left out.
template <int NV>
struct LabelledRegRow {
  typedef float data_type;
  const RegRow<float, NV>* row;
  int y;
  __device__ __forceinline__ int size() const { return row->m - 1; }
  template <typename F>
  __device__ __forceinline__ void for_each(F&& f) const {
    row->for_each([&](float x, int i) { if (i != y) f(x, i); });
  }
};

// s -> h in place; returns this lane's share of #{j != y : s_j >= s_y}.
template <int NV>
__device__ __forceinline__ int shift_row_and_count(RegRow<float, NV>& row, int y, float sy, int lane) {
  const float shift = 1.0f - sy;
  int r = 0;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int base = (j * 32 + lane) * 4;
    float* e = reinterpret_cast<float*>(&row.v[j]);
    if (base < row.m) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const bool label = (base + c == y);
        r += (!label && e[c] >= sy) ? 1 : 0;
        e[c] = label ? -num<float>::inf() : e[c] + shift;
      }
    }
  }
  return r;
}

template <typename R, int NV, bool SMOOTH>
__global__ void __launch_bounds__(kLossThreads)
eval_loss_rows_kernel(LossArgs g, const float* __restrict__ scores, const float* __restrict__ A,
                      double* __restrict__ block_partials, unsigned long long* __restrict__ hist) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ double warp_sums[kLossThreads / 32][4];
  __shared__ unsigned int local_hist[kHistLocal];
  __shared__ float slots_all[SMOOTH ? kLossThreads / 32 : 1][32];
  __shared__ int counters[kLossThreads / 32];
  __shared__ R sorted_all[SMOOTH ? kLossThreads / 32 : 1][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = kLossThreads / 32;
  float* stage = reinterpret_cast<float*>(smem_raw) + static_cast<size_t>(warp) * g.m_pad;
  for (int i = threadIdx.x; i < kHistLocal; i += kLossThreads) local_hist[i] = 0;
  if (lane == 0) counters[warp] = 0;
  __syncthreads();
  const int m = g.m, k = g.obj.k;
  const R gamma = static_cast<R>(g.obj.gamma);
  const TopkConsts<R> tc(k > 0 ? k : 1, SMOOTH ? gamma : R(1), R(0));
  double primal = 0, dual = 0;
  for (long long e = static_cast<long long>(blockIdx.x) * warps + warp; e < g.n;
       e += static_cast<long long>(gridDim.x) * warps) {
    const float* s_g = scores + e * m;
    const long long ex = g.first + e;
    const int y = static_cast<int>(g.labels[ex]);
    const float sy = s_g[y];
    RegRow<float, NV> row;
    row.m = m;
    row.load_keep(s_g, lane);
    const int rank = warp_sum(shift_row_and_count<NV>(row, y, sy, lane));
    if (lane == 0) {
      if (rank < kHistLocal) atomicAdd(&local_hist[rank], 1u);
      else atomicAdd(&hist[rank], 1ull);
    }
    if (!SMOOTH) {
      LabelledRegRow<NV> h{&row, y};
      R sum_all, sum_pos;
      topk_sums<R>(h, k, sum_all, sum_pos);
      primal += static_cast<double>((g.obj.id == kObjL2HingeTopk) ? max_(R(0), sum_all) : sum_pos);
    } else {
      Thr<R> thr;
      const FastStatus st = fast_topk_simplex<R>(row, k, gamma, R(0), tc, slots_all[warp], &counters[warp],
                                                 sorted_all[warp], lane, thr);
      if (st == kFastDone) {
        // the search is over: the row again (an L2 hit), for the sums over the sets
        RegRow<float, NV> again;
        again.m = m;
        again.load(s_g, lane);
        shift_row_and_count<NV>(again, y, sy, lane);
        LabelledRegRow<NV> h{&again, y};
        primal += static_cast<double>(smooth_loss_from_thresholds<R>(h, thr));
      } else {
        for (int i = lane; i < m; i += 32) stage[i] = s_g[i];
        __syncwarp();
        int unused;
        primal += static_cast<double>(multiclass_primal_loss<R, float>(g.obj, stage, m, y, unused));
        __syncwarp();
      }
    }
    if (g.is_train && A) {
      const float* a = A + (g.a_row_offset + ex) * m;
      if (!SMOOTH) {
        dual += static_cast<double>(static_cast<R>(a[y]));      // objective_base.h:49-56
      } else {
        // l2_hinge_topk.h:182-192: a_y - gamma / (2 c) sum_{j != y} a_j^2
        RegRow<float, NV> ar;
        ar.m = m;
        ar.load(a, lane);
        R dot = 0;
        ar.for_each([&](float x, int i) {
          const R v = static_cast<R>(x);
          if (i != y) dot += v * v;
        });
        dot = warp_sum(dot);
        dual += static_cast<double>(static_cast<R>(a[y]) - gamma / (R(2) * static_cast<R>(g.obj.c)) * dot);
      }
    }
  }
  if (lane == 0) {
    warp_sums[warp][0] = primal; warp_sums[warp][1] = dual;
    warp_sums[warp][2] = 0; warp_sums[warp][3] = 0;
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

// Whether a launch qualifies: multiclass top-k hinge (alpha or beta, gamma = 0: k <= 8, the
// sizes topk_sums keeps in registers) or the smooth alpha form, features, rows of 64 to
// 1024 floats in whole 16-byte vectors, aligned.
inline bool loss_rows_usable(const LossArgs& g, const float* scores, const float* A) {
  const int id = g.obj.id;
  const bool hinge = (id == kObjL2HingeTopk || id == kObjL2TopkHinge) && g.obj.k >= 1 && g.obj.k <= 8;
  const bool smooth = (id == kObjL2HingeTopkSmooth) && g.obj.k >= 1 && g.obj.k <= 31;
  if (!hinge && !smooth) return false;
  if (g.kernel_input || g.m % 4 != 0 || g.m < 64 || g.m > 1024 || g.obj.k >= g.m - 1) return false;
  if (reinterpret_cast<uintptr_t>(scores) & 15) return false;
  if (g.is_train && A && (reinterpret_cast<uintptr_t>(A) & 15)) return false;
  return true;
}
inline bool loss_rows_usable(const LossArgs&, const double*, const double*) { return false; }

template <typename R>
int launch_loss_rows(const LossArgs& g, const float* scores, const float* A, double* partials,
                     unsigned long long* hist, int blocks, size_t smem_optin, cudaStream_t stream) {
  const bool smooth = (g.obj.id == kObjL2HingeTopkSmooth);
  const int vecs = (g.m + 3) / 4;
  const size_t smem = smooth ? static_cast<size_t>(kLossThreads / 32) * g.m_pad * sizeof(float) : 0;
  if (smem > smem_optin) return SDCAB_ERR_TOO_LARGE;
#define SDCAB_LOSS_ROWS(NVV, SM)                                                                   \
  do {                                                                                             \
    auto kernel = eval_loss_rows_kernel<R, NVV, SM>;                                               \
    if (smem > 48 * 1024)                                                                          \
      SDCAB_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                          static_cast<int>(smem)));                                \
    kernel<<<blocks, kLossThreads, smem, stream>>>(g, scores, A, partials, hist);                  \
  } while (0)
  if (vecs <= 64) { if (smooth) SDCAB_LOSS_ROWS(2, true); else SDCAB_LOSS_ROWS(2, false); }
  else if (vecs <= 128) { if (smooth) SDCAB_LOSS_ROWS(4, true); else SDCAB_LOSS_ROWS(4, false); }
  else { if (smooth) SDCAB_LOSS_ROWS(8, true); else SDCAB_LOSS_ROWS(8, false); }
#undef SDCAB_LOSS_ROWS
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}
}  // namespace sdcab
