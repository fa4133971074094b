// two_simplex_sort: the sort-based solver of
//     min ||x - a||^2 + ||y - b||^2   s.t.  <1, x> = <1, y> <= rhs,  x, y >= 0
// that matsdca_prox offers beside two_simplex
// (include/sdca/prox/two_simplex_sort.h:24-111 of the reference, after the
// bipartite solver of Shalev-Shwartz's Sopopo).  It is not the same function as
// two_simplex: it starts from one active entry in each block and a common sum
// c >= 0, walks the grid of sums at which a further entry of either block
// becomes active, and clips at hi = rhs; on inputs where the variable-fixing
// solver ends with an empty block or a zero sum the two differ.  A drop-in has to
// reproduce this routine under this name, so it is restated here step by step.
//
// One warp per row.  The walk usually ends after a few entries of each block, so it is first
// given only the largest entries of each block (everything at or above the eighth largest
// lane maximum, ordered by one shuffle network); when it asks for an entry beyond those, both
// blocks are sorted in descending order in shared memory (bitonic network over the next power
// of two, padded with -inf) and the walk runs again.  Either way one lane walks the grid
// exactly as the reference does -- the same running sums in the same order, so
// double-precision results agree to the last bit -- and the warp applies
// max(0, min(a - theta, rhs))  to the unsorted row.
#pragma once

#include "prox_core.cuh"
#ifdef __CUDACC__
#include "fast_rows.cuh"   // kth_largest_of_lanes, the one-value-per-lane sort
#endif

namespace sdcab {

constexpr int kSortThreads = 128;

SDCAB_HD int pow2_ceil(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

// The walk of two_simplex_sort.h:46-103 on the sorted blocks a[0 .. na), b[0 .. nb).
// a and b may hold only the avail_a / avail_b largest entries of their blocks (the whole block when
// avail == n): the walk then returns false as soon as it needs an entry beyond what it was given,
// having computed exactly what it would have computed on the full arrays up to that point.
template <typename R, typename Data>
SDCAB_HD bool two_simplex_sort_walk(const Data* a, int na, const Data* b, int nb, R rhs,
                                    R& theta_a, R& theta_b, int& r_out, int& s_out,
                                    int avail_a = -1, int avail_b = -1) {
  if (avail_a < 0) avail_a = na;
  if (avail_b < 0) avail_b = nb;
  if (avail_a < 1 || avail_b < 1 || (avail_a < 2 && na > 1) || (avail_b < 2 && nb > 1)) return false;
  const R one = R(1);
  const R eps = num<R>::eps() * (one < rhs ? rhs : one);
  R c = 0, best_c = rhs;
  const R C = rhs;
  R sum_mu = static_cast<R>(a[0]), sum_nu = static_cast<R>(b[0]);
  int r = 1, s = 1;
  // pseudo points beyond the ends make the walk terminate
  R a_r = (r != na) ? static_cast<R>(a[r]) : static_cast<R>(a[na - 1]) - C;
  R b_s = (s != nb) ? static_cast<R>(b[s]) : static_cast<R>(b[nb - 1]) - C;
  while (c < C) {
    const R copt = (static_cast<R>(s) * sum_mu + static_cast<R>(r) * sum_nu) / static_cast<R>(r + s);
    const R next_cr = (sum_mu + a_r) - static_cast<R>(r + 1) * a_r;
    const R next_cs = (sum_nu + b_s) - static_cast<R>(s + 1) * b_s;
    R next_c = next_cr < next_cs ? next_cr : next_cs;   // std::min(std::min(cr, cs), C)
    next_c = C < next_c ? C : next_c;
    if (c <= copt && copt < next_c) { best_c = copt; break; }
    if (next_c >= C - eps) { best_c = C; break; }
    // A block that is used up offers its pseudo point, whose grid value is C in exact
    // arithmetic, so the test above ends the walk there.  When rounding puts that
    // value a few ulps below C the reference steps over the pseudo point and reads
    // past the end of the block (its result is then whatever follows in memory);
    // here the walk ends with the sum the exact arithmetic gives.
    if (next_cr < next_cs ? (r == na) : (s == nb)) { best_c = C; break; }
    if (next_cr < next_cs) {
      sum_mu += a_r; ++r;
      if (r != na && r >= avail_a) return false;
      a_r = (r != na) ? static_cast<R>(a[r]) : static_cast<R>(a[na - 1]) - C;
    } else {
      sum_nu += b_s; ++s;
      if (s != nb && s >= avail_b) return false;
      b_s = (s != nb) ? static_cast<R>(b[s]) : static_cast<R>(b[nb - 1]) - C;
    }
    c = next_c;
  }
  theta_a = (sum_mu - best_c) / static_cast<R>(r);
  theta_b = (sum_nu - best_c) / static_cast<R>(s);
  r_out = r; s_out = s;
  return true;
}

#ifdef __CUDACC__
// Descending bitonic sort of buf[0 .. len) (len a power of two) by one warp.
template <typename Data>
__device__ void warp_sort_desc(Data* buf, int len, int lane) {
  for (int k = 2; k <= len; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = lane; i < len; i += 32) {
        const int partner = i ^ j;
        if (partner > i) {
          const Data x = buf[i], y = buf[partner];
          const bool descending = ((i & k) == 0);
          if (descending ? (x < y) : (x > y)) { buf[i] = y; buf[partner] = x; }
        }
      }
      __syncwarp();
    }
  }
}

// The largest entries of a block of more than 32 entries, in descending order, into dst[0 .. 32):
// everything at or above the eighth largest lane maximum (so at least eight entries).  Returns
// their number, or -1 when more than 32 qualify.  *counter is 0 on entry and on return.
template <typename Data>
__device__ __forceinline__ int block_top_entries(const Data* __restrict__ g, int len, int lane,
                                                 Data* dst, Data* slots, int* counter) {
  Data lm = -num<Data>::inf();
  for (int i = lane; i < len; i += 32) lm = max_(lm, g[i]);
  const Data tau = kth_largest_of_lanes(lm, 7, lane);
  for (int i = lane; i < len; i += 32) {
    const Data x = g[i];
    if (x >= tau) {
      const int pos = atomicAdd(counter, 1);
      if (pos < 32) slots[pos] = x;
    }
  }
  __syncwarp();
  const int total = *counter;
  Data v = (lane < total && total <= 32) ? slots[lane] : -num<Data>::inf();
  __syncwarp();
  if (lane == 0) *counter = 0;
  __syncwarp();
  if (total > 32) return -1;
  v = warp_sort_desc(v, lane);
  dst[lane] = v;
  __syncwarp();
  return total;
}

// smem per warp: pa + pb elements of Data, pa = pow2_ceil(p), pb = pow2_ceil(m - p)
template <typename Data, typename R>
__global__ void __launch_bounds__(kSortThreads)
two_simplex_sort_kernel(const Data* a, Data* out, int m, long long n, ProxParams q,
                        sdcab_thresholds* __restrict__ thr_out, int apply, int pa, int pb) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ Data slots_all[kSortThreads / 32][32];
  __shared__ int counters[kSortThreads / 32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  if (lane == 0) counters[warp] = 0;
  __syncwarp();
  Data* sa = reinterpret_cast<Data*>(smem_raw) + static_cast<size_t>(warp) * (pa + pb);
  Data* sb = sa + pa;
  const int p = q.p;
  const Data neg_inf = -num<Data>::inf();
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + warp; row < n;
       row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const Data* gin = a + row * m;
    Data* g = out + row * m;
    R ta = 0, tb = 0;
    int r = 0, s = 0;
    // The walk usually ends after a few entries of each block: give it the largest entries
    // only (found without sorting the blocks) and sort the whole blocks when it asks for more.
    int complete = 0;
    if (p > 32 && m - p > 32) {
      const int la = block_top_entries(gin, p, lane, sa, slots_all[warp], &counters[warp]);
      const int lb = (la > 0) ? block_top_entries(gin + p, m - p, lane, sb, slots_all[warp], &counters[warp]) : -1;
      if (la > 0 && lb > 0) {
        if (lane == 0)
          complete = two_simplex_sort_walk<R, Data>(sa, p, sb, m - p, static_cast<R>(q.rhs), ta, tb, r, s, la, lb) ? 1 : 0;
        complete = __shfl_sync(0xffffffffu, complete, 0);
      }
      __syncwarp();
    }
    if (!complete) {
      for (int i = lane; i < pa; i += 32) sa[i] = (i < p) ? gin[i] : neg_inf;
      for (int i = lane; i < pb; i += 32) sb[i] = (i < m - p) ? gin[p + i] : neg_inf;
      __syncwarp();
      warp_sort_desc(sa, pa, lane);
      warp_sort_desc(sb, pb, lane);
      if (lane == 0) two_simplex_sort_walk<R, Data>(sa, p, sb, m - p, static_cast<R>(q.rhs), ta, tb, r, s);
    }
    ta = __shfl_sync(0xffffffffu, ta, 0);
    tb = __shfl_sync(0xffffffffu, tb, 0);
    r = __shfl_sync(0xffffffffu, r, 0);
    s = __shfl_sync(0xffffffffu, s, 0);
    if (thr_out && lane == 0) {
      sdcab_thresholds o;
      o.lo = 0; o.hi = q.rhs; o.num_hi = 0; o.reserved = 0;
      o.t = ta; o.num_mid = r; o.status = finite_(ta) ? kThrSolved : kThrNotFinite; thr_out[2 * row] = o;
      o.t = tb; o.num_mid = s; o.status = finite_(tb) ? kThrSolved : kThrNotFinite; thr_out[2 * row + 1] = o;
    }
    if (apply) {
      const Thr<R> tha = make_thr(ta, R(0), static_cast<R>(q.rhs), 0, 0, R(0), R(0));
      const Thr<R> thb = make_thr(tb, R(0), static_cast<R>(q.rhs), 0, 0, R(0), R(0));
      Applier<Data> fa(tha, kMapIdentity, 1.0), fb(thb, kMapIdentity, 1.0);
      for (int i = lane; i < m; i += 32) {
        const Data v = gin[i];
        g[i] = (i < p) ? fa(v) : fb(v);
      }
    }
    __syncwarp();
  }
}

#endif  // __CUDACC__

}  // namespace sdcab
