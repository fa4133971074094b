// Entropic projections of float rows with the scalar work batched over rows.
//
// The entropy and top-k entropy projections (include/sdca/prox/entropy.h:19-53,
// include/sdca/prox/topk_entropy.h:20-76 of the reference) reduce a row to a
// handful of numbers -- its maximum, the sum of exponentials, for the top-k
// form the k + 1 largest entries -- and then spend several hundred
// instructions of double-precision logarithms and exponentials on those
// numbers.  With one warp per row that scalar work runs once per row on all 32
// lanes with one lane's worth of result.  Here a block takes a group of up to
// 32 consecutive rows and works in three phases:
//   A  one warp per row: maximum, sum of exponentials, candidates (the row is
//      read with ld.global.cg, so that it stays in L2);
//   B  one warp, one lane per row: the closed forms for t and hi of all rows of
//      the group at the same time;
//   C  one warp per row: the row is read again (an L2 hit), mapped and stored.
// The group size is chosen so that the rows all resident blocks hold between A
// and C stay well inside L2.
#pragma once

#include "fast_rows.cuh"

namespace sdcab {

// Bytes of rows that all resident blocks together hold between phases A and C
// (32 MB and more measured equal on a 126 MB L2, less was slower).
#ifndef SDCAB_GROUP_FOOTPRINT
#define SDCAB_GROUP_FOOTPRINT (32ll << 20)
#endif
// Resident blocks per SM the register allocation aims for.
#ifndef SDCAB_GROUP_MIN_BLOCKS
#define SDCAB_GROUP_MIN_BLOCKS 8
#endif
constexpr int kGroupMaxRows = 32;
constexpr int kGroupMinRows = 8;

// Scratch of one group.  `cand` is padded to 33 columns so that the
// lanes of phase B, each walking its own row, hit different banks.
template <typename R, bool WITH_CAND>
struct GroupScratch {
  R sum_or_t[kGroupMaxRows];      // phase A: sum of exponentials; phase B: t
  R hi[kGroupMaxRows];
  float mx[kGroupMaxRows];
  int total[kGroupMaxRows];       // phase A: number of candidates; phase B: < 0 = general routine
  float cand[WITH_CAND ? kGroupMaxRows : 1][33];
};

template <typename R>
struct GroupResult {
  R t, hi;
  bool full;
};

// The k largest entries of a row held NV vectors per lane, in descending order, one per
// lane (lane r gets the r-th largest, lanes >= k get -inf; k <= 32).  Every lane orders
// its own entries with a sorting network; then k rounds pop the largest head: one
// redux.sync.max over the heads, and the first lane that holds it moves its list up.
// Repeated values are popped one per round, as a sort of the whole row would list them.
__device__ __forceinline__ void order_pair(float& a, float& b) {
  const float hi = fmaxf(a, b), lo = fminf(a, b);
  a = hi; b = lo;
}
template <int N>
__device__ __forceinline__ void sort_desc_in_lane(float (&h)[N]) {
  if constexpr (N == 8) {
    // the 19-exchange network for eight inputs
    order_pair(h[0], h[1]); order_pair(h[2], h[3]); order_pair(h[4], h[5]); order_pair(h[6], h[7]);
    order_pair(h[0], h[2]); order_pair(h[1], h[3]); order_pair(h[4], h[6]); order_pair(h[5], h[7]);
    order_pair(h[1], h[2]); order_pair(h[5], h[6]); order_pair(h[0], h[4]); order_pair(h[3], h[7]);
    order_pair(h[1], h[5]); order_pair(h[2], h[6]);
    order_pair(h[1], h[4]); order_pair(h[3], h[6]);
    order_pair(h[2], h[4]); order_pair(h[3], h[5]);
    order_pair(h[3], h[4]);
  } else {
    // bitonic network, N a power of two
#pragma unroll
    for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
      for (int j = k >> 1; j > 0; j >>= 1) {
#pragma unroll
        for (int i = 0; i < N; ++i) {
          const int l = i ^ j;
          if (l > i) {
            if ((i & k) == 0) order_pair(h[i], h[l]);
            else order_pair(h[l], h[i]);
          }
        }
      }
    }
  }
}
template <int NV>
__device__ __forceinline__ float largest_k_of_row(const RegRow<float, NV>& row, int k, int lane) {
  constexpr int N = NV * 4;
  float h[N];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const float* e = reinterpret_cast<const float*>(&row.v[j]);   // vectors past the end hold -inf
#pragma unroll
    for (int c = 0; c < 4; ++c) h[j * 4 + c] = e[c];
  }
  sort_desc_in_lane<N>(h);
  float mine = -num<float>::inf();
  for (int r = 0; r < k; ++r) {
    const float top = warp_max_fast(h[0]);
    const unsigned hit = __ballot_sync(kFullMask, h[0] == top);
    if (lane == r) mine = top;
    if (lane == __ffs(hit) - 1) {
#pragma unroll
      for (int j = 0; j + 1 < N; ++j) h[j] = h[j + 1];
      h[N - 1] = -num<float>::inf();
    }
  }
  return mine;
}

// Phase B of the top-k entropy projection for one row: the same closed forms as
// fast_topk_entropy, the sizes of U tried one after the other by this lane.
template <typename R>
__device__ __forceinline__ GroupResult<R> grouped_topk_entropy(R S, float mxf, int total,
                                                               float* cand, int k,
                                                               const R* log_of) {
  GroupResult<R> out;
  out.full = false;
  const R eps = 16 * num<R>::eps();
  const R K = static_cast<R>(k);
  const R mx = static_cast<R>(mxf);
  const R z = max_(S - R(1), R(0));
  const R log_z = mx + log1p_(z);
  if (k <= 1 || mx - eps <= log_z - log_of[k]) {
    const R e = exp_(-mx);
    out.t = finite_(e) ? mx + log1p_(z + e) : R(0);
    out.hi = R(1);
    return out;
  }
  // a row with a NaN has a NaN sum; its candidates are not ordered: the general routine
  if (total <= k || !(S == S)) {
    out.full = true;
    return out;
  }
  const int last = k - 1;
  const float top = cand[0];
  R pe_prev = static_cast<R>(exp_(top - mxf));       // sum of the exponentials of U
  R s_prev = static_cast<R>(top);                    // smallest entry of U
  R sum_U = s_prev;
  R zs = 0, log_zs = 0, cur_max = 0;
  int ustar = last;
  for (int u = 1; u <= last; ++u) {
    const float sf = cand[u];
    const R s = static_cast<R>(sf);
    const R rest = S - pe_prev;                      // relative to the old maximum
    // a rest that is a small fraction of the whole sum has lost too many digits
    if (!(rest > R(1e-3) * S)) { out.full = true; return out; }
    zs = max_(rest * exp_(mx - s) - R(1), R(0));
    log_zs = s + log1p_(zs);
    cur_max = s;
    ustar = u;
    const R tt = log_zs - log_of[k - u];
    if ((s - eps <= tt && tt <= s_prev + eps) || u == last) break;
    pe_prev += static_cast<R>(exp_(sf - mxf));
    sum_U += s;
    s_prev = s;
  }
  const R k_u = K - static_cast<R>(ustar);
  const R tmp = ((K - k_u) * log_zs + k_u * log_of[k - ustar] - sum_U) / K;
  if (tmp > cur_max) {
    const R a = (1 + zs) * exp_(cur_max - tmp);
    out.t = tmp + log1p_(a * K) - log_of[k - ustar];
    out.hi = a / (1 + a * K);
  } else {
    const R a = exp_(tmp - cur_max) / K;
    out.t = cur_max + log1p_(zs + a) - log_(k_u / K);
    out.hi = (1 + zs) / ((1 + zs + a) * K);
  }
  return out;
}

template <typename R, int PROX, int NV>
__global__ void __launch_bounds__(kFastThreads, SDCAB_GROUP_MIN_BLOCKS)
entropic_grouped_kernel(const float* a, float* out, int m, long long n,
                        ProxParams q, int m_pad, int group) {
  constexpr bool kTopkForm = (PROX == kTopkEntropy);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ GroupScratch<R, kTopkForm> sc;
  __shared__ R log_of[33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps_per_block = kFastThreads / 32;
  if (threadIdx.x < 33) log_of[threadIdx.x] = threadIdx.x ? log_(static_cast<R>(threadIdx.x)) : R(0);
  __syncthreads();
  float* stage = reinterpret_cast<float*>(smem_raw) + static_cast<size_t>(warp) * m_pad;
  const int k = q.k;
  const R rhs = static_cast<R>(q.rhs), hi_bound = static_cast<R>(q.hi);
  const R log_rhs = kTopkForm ? R(0) : log_(rhs);
  const R log_hi = kTopkForm ? R(0) : log_(hi_bound);
  // sum of exponentials above which the plain entropy case is certain
  const R certain = static_cast<R>(k) * (R(1) + R(1e-6));
  const long long groups = (n + group - 1) / group;
  // every thread of the block runs the same number of iterations (barriers inside)
  for (long long g = blockIdx.x; g < groups; g += gridDim.x) {
    const long long r0 = g * group;
    const int cnt = static_cast<int>(min(static_cast<long long>(group), n - r0));
    // phase A: the rows of the group dealt out to the warps.  A row's scratch entries
    // are written and, in phase C, read by the same warp, so the next group's phase A
    // needs no barrier after phase C.
    for (int i = warp; i < cnt; i += warps_per_block) {
      RegRow<float, NV> row;
      row.m = m;
      row.load_keep(a + (r0 + i) * m, lane);
      float mxf, lm;
      R S;
      row_max_and_expsum<R, NV>(row, mxf, lm, S);
      int total = 0;
      if (kTopkForm && k > 1 && !(S > certain)) {
        // the k largest entries in descending order, for phase B
        sc.cand[kTopkForm ? i : 0][lane] = largest_k_of_row<NV>(row, k, lane);
        total = k + 1;
      }
      if (lane == 0) {
        sc.sum_or_t[i] = S;
        sc.mx[i] = mxf;
        sc.total[i] = total;
      }
    }
    __syncthreads();
    // phase B: one warp, one lane per row; the other warps wait at the barrier, which
    // costs no issue slots (the other resident blocks use them)
    if (warp == static_cast<int>(g % warps_per_block) && lane < cnt) {
      const R S = sc.sum_or_t[lane];
      const float mxf = sc.mx[lane];
      GroupResult<R> res;
      if (kTopkForm) {
        res = grouped_topk_entropy<R>(S, mxf, sc.total[lane], sc.cand[kTopkForm ? lane : 0], k, log_of);
      } else {
        // include/sdca/prox/entropy.h:19-53 when no entry reaches the upper bound
        const R eps = 16 * num<R>::eps() * max_(R(1), rhs);
        const R mx = static_cast<R>(mxf);
        res.t = (mx + log1p_(max_(S - R(1), R(0)))) - log_rhs;
        res.hi = hi_bound;
        res.full = mx > res.t + log_hi + eps;
      }
      sc.sum_or_t[lane] = res.t;
      sc.hi[lane] = res.hi;
      sc.total[lane] = res.full ? -1 : 0;
    }
    __syncthreads();
    // phase C
    for (int i = warp; i < cnt; i += warps_per_block) {
      const float* src = a + (r0 + i) * m;
      RegRow<float, NV> row;
      row.m = m;
      row.load(src, lane);
      Thr<R> thr;
      if (sc.total[i] < 0) {
        row.for_each([&](float x, int j) { stage[j] = x; });
        __syncwarp();
        thr = full_row_thresholds<R, float, PROX>(stage, m, &q);
        __syncwarp();
      } else {
        thr = make_thr(sc.sum_or_t[i], R(0), sc.hi[i], 0, m, num<R>::inf(), -num<R>::inf());
      }
      Applier<float> f(thr, prox_map(PROX), q.alpha);
      row.store(out + (r0 + i) * m, lane, f);
    }
  }
}

template <typename R, int PROX, int NV>
int launch_entropic_grouped(const float* a, float* out, int m, long long n, const ProxParams& q,
                            cudaStream_t stream) {
  DeviceInfo info;
  int rc = get_device_info(&info);
  if (rc) return rc;
  auto kernel = entropic_grouped_kernel<R, PROX, NV>;
  const int m_pad = (m + 15) & ~15;
  const int warps = kFastThreads / 32;
  const size_t smem = static_cast<size_t>(warps) * m_pad * sizeof(float);
  int per_sm = 0;
  SDCAB_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kFastThreads, smem));
  if (per_sm < 1) per_sm = 1;
  const long long resident = static_cast<long long>(per_sm) * info.sm_count;   // blocks
  long long group = SDCAB_GROUP_FOOTPRINT / (resident * m * static_cast<long long>(sizeof(float)));
  group = std::min<long long>(group, n / resident);      // every resident block gets a group
  group = std::min<long long>(group, kGroupMaxRows);
  if (group < kGroupMinRows) return kNoFastPath;
  const long long groups = (n + group - 1) / group;
  const int blocks = static_cast<int>(std::max<long long>(1, std::min<long long>(groups, resident)));
  kernel<<<blocks, kFastThreads, smem, stream>>>(a, out, m, n, q, m_pad, static_cast<int>(group));
  SDCAB_CUDA_TRY(cudaGetLastError());
  return SDCAB_OK;
}

// Float rows of the entropy and top-k entropy projections that qualify for the
// grouped kernel; kNoFastPath hands the launch to the one-warp-per-row kernel.
template <typename R>
int launch_entropic_rows(int prox, const float* a, float* out, int m, long long n,
                         const ProxParams& q, cudaStream_t stream) {
  if (prox != kEntropy && prox != kTopkEntropy) return kNoFastPath;
  if (prox == kTopkEntropy && (q.k > 30 || m <= 32 || q.k > m)) return kNoFastPath;
  const int vecs = (m + 3) / 4;
#define SDCAB_GROUPED(NVV)                                                                       \
  return prox == kEntropy ? launch_entropic_grouped<R, kEntropy, NVV>(a, out, m, n, q, stream)   \
                          : launch_entropic_grouped<R, kTopkEntropy, NVV>(a, out, m, n, q, stream)
  // longer rows never reach the smallest useful group within the L2 budget
  if (vecs <= 32 * 2) { SDCAB_GROUPED(2); }
  if (vecs <= 32 * 4) { SDCAB_GROUPED(4); }
#undef SDCAB_GROUPED
  return kNoFastPath;
}

}  // namespace sdcab
