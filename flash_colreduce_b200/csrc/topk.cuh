// Row-wise top-k selection over the (B*H, N) score array the column reduction
// produces: the step a token-pruning consumer runs next (the reference's
// README.md:9 names that use; the reference itself stops at the scores, so this
// kernel has no counterpart there).
//
// One thread-block cluster per row: a single CTA when there are enough rows to
// fill the GPU (256 threads when the rows are short and many, so that several
// rows share an SM), otherwise 2, 4 or 8 CTAs that each own a contiguous slice of the
// row and exchange their 256-bin histograms and their selected-element counts
// through distributed shared memory (cluster.sync() is a hardware barrier, there
// is no spin wait).  The k-th largest value is found by a most-significant-byte
// first radix select on an order-preserving key (four histogram rounds for fp32
// scores, two for fp16 / bf16, each a sweep over the row, which stays in the L2
// cache; one histogram per lane, so skewed scores cause no shared-memory
// conflicts), then one more sweep compacts the selected positions in ascending
// index order with a block-wide scan: every element above the threshold, plus
// the first `ties` elements equal to it.  Deterministic; a NaN with a clear sign
// bit (the 0/0 of an empty mean) orders above +inf, as in torch.topk.
//
// Included by colreduce_sm100.cu (needs FCR_F16 / FCR_BF16 / FCR_F32).
#pragma once
#include <cooperative_groups.h>

namespace fcr {

constexpr int kTopkThreads = 1024;      // long rows: one CTA (or a cluster of CTAs) of 1024 threads per row
constexpr int kTopkThreadsSmall = 256;  // many short rows: 256 threads per row, up to eight rows per SM at a time
constexpr int kTopkItems = 8;  // consecutive elements per thread and sweep step (one 16-byte load for 16-bit scores)

// Order-preserving unsigned key of a score: 32 bits for fp32, 16 bits for fp16 / bf16 (both are
// sign-magnitude formats, so the same bit trick orders them), hence two radix rounds instead of four.
template <typename T>
struct TopkKey;
template <>
struct TopkKey<float> {
  static constexpr int kBits = 32;
  static __device__ __forceinline__ uint32_t of(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  }
};
template <>
struct TopkKey<__half> {
  static constexpr int kBits = 16;
  static __device__ __forceinline__ uint32_t of(__half x) {
    const uint32_t u = __half_as_ushort(x);
    return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
  }
};
template <>
struct TopkKey<__nv_bfloat16> {
  static constexpr int kBits = 16;
  static __device__ __forceinline__ uint32_t of(__nv_bfloat16 x) {
    const uint32_t u = __bfloat16_as_ushort(x);
    return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
  }
};

// Keys of elements [i0, i0 + 8) of a row (unspecified beyond n); 16-byte loads when the address allows.
template <typename T>
__device__ __forceinline__ void topk_load8(const T* row, int i0, int n, uint32_t (&key)[kTopkItems]) {
  const T* p = row + i0;
  if (i0 + kTopkItems <= n && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
    constexpr int kVecs = (int)(kTopkItems * sizeof(T) / 16);
    uint4 raw[kVecs];
#pragma unroll
    for (int v = 0; v < kVecs; ++v) raw[v] = reinterpret_cast<const uint4*>(p)[v];
    const T* e = reinterpret_cast<const T*>(raw);
#pragma unroll
    for (int j = 0; j < kTopkItems; ++j) key[j] = TopkKey<T>::of(e[j]);
  } else {
#pragma unroll
    for (int j = 0; j < kTopkItems; ++j) key[j] = (i0 + j < n) ? TopkKey<T>::of(p[j]) : 0u;
  }
}

// THREADS: 1024 or 256.  COPIES: histogram copies, indexed by lane & (COPIES - 1): 32 make a warp's
// adds conflict-free, 8 keep the histogram at 8 KB for the small blocks (at most 4 lanes per word).
template <typename T, typename IndexT, int THREADS, int COPIES>
__global__ void __launch_bounds__(THREADS)
topk_kernel(const T* __restrict__ scores, int n, int k, IndexT* __restrict__ indices,
            T* __restrict__ values) {
  static_assert(THREADS >= 256 && THREADS <= 1024 && THREADS % 32 == 0, "256 bins need 256 threads; one warp scans the warp totals");
  constexpr int kTopkThreads = THREADS;  // shadows the namespace constant inside the kernel
  constexpr int kWarps = THREADS / 32;
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int n_ranks = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  // One histogram per lane (COPIES = 32): hist[bin * 32 + lane].  A warp's 32 adds then touch 32
  // different banks and never the same word, however skewed the scores are.
  __shared__ int hist[256 * COPIES];
  __shared__ int bin_total[256];     // this CTA's slice, read by the other CTAs of the cluster
  __shared__ uint32_t slice_cnt[2];  // elements above / equal to the threshold in this CTA's slice
  __shared__ uint32_t s_prefix, s_want;
  __shared__ uint32_t warp_tot[kTopkThreads / 32];
  __shared__ uint32_t chunk_tot;
  const size_t row_id = blockIdx.x / n_ranks;
  const T* row = scores + row_id * n;
  IndexT* out_idx = indices + row_id * k;
  T* out_val = values ? values + row_id * k : nullptr;
  const int tid = (int)threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kStep = kTopkThreads * kTopkItems;
  // this CTA's slice [lo, hi) of the row; inner boundaries are multiples of 8 elements
  const int lo = (int)(((long long)n * rank / n_ranks) & ~7LL);
  const int hi = rank + 1 == n_ranks ? n : (int)(((long long)n * (rank + 1) / n_ranks) & ~7LL);

  // ---- radix select: after the last round `prefix` is the key of the k-th largest element
  uint32_t prefix = 0, mask = 0, want = (uint32_t)k;
  for (int shift = TopkKey<T>::kBits - 8; shift >= 0; shift -= 8) {
#pragma unroll
    for (int j = 0; j < 256 * COPIES / kTopkThreads; ++j) hist[j * kTopkThreads + tid] = 0;
    __syncthreads();
    for (int c0 = lo; c0 < hi; c0 += kStep) {
      const int i0 = c0 + tid * kTopkItems;
      uint32_t key[kTopkItems];
      topk_load8<T>(row, i0, hi, key);
#pragma unroll
      for (int j = 0; j < kTopkItems; ++j) {
        if (i0 + j < hi && (key[j] & mask) == prefix)
          atomicAdd(&hist[((key[j] >> shift) & 255u) * COPIES + (lane & (COPIES - 1))], 1);
      }
    }
    __syncthreads();
    // bin totals (thread b sums the 32 copies of bin b, starting at its own lane: no bank conflicts)
    if (tid < 256) {
      int total = 0;
#pragma unroll
      for (int j = 0; j < COPIES; ++j) total += hist[tid * COPIES + ((j + lane) & (COPIES - 1))];
      bin_total[tid] = total;
    }
    cluster.sync();  // every slice's totals are complete (also a barrier of this CTA)
    if (warp == 0) {
      // lane L owns bins [8L, 8L + 8), summed over the slices; `above` = elements in higher bins
      uint32_t bins[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) bins[j] = 0;
      for (int r = 0; r < n_ranks; ++r) {
        const int* remote = cluster.map_shared_rank(bin_total, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) bins[j] += (uint32_t)remote[lane * 8 + j];
      }
      uint32_t mine = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) mine += bins[j];
      uint32_t suffix = mine;  // inclusive sum over lanes >= L
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t dn = __shfl_down_sync(0xffffffffu, suffix, d);
        if (lane + d < 32) suffix += dn;
      }
      uint32_t above = suffix - mine;
      if (above < want && want <= suffix) {  // the wanted element lies in one of this lane's bins
        int j = 7;
#pragma unroll
        for (int u = 7; u > 0; --u) {
          if (j == u && above + bins[u] < want) {
            above += bins[u];
            j = u - 1;
          }
        }
        s_prefix = prefix | ((uint32_t)(lane * 8 + j) << shift);
        s_want = want - above;  // how many elements of that bin are still needed
      }
    }
    cluster.sync();  // the totals have been read everywhere: they may be rebuilt in the next round
    prefix = s_prefix;
    want = s_want;
    mask |= 255u << shift;
  }
  const uint32_t thr = prefix;  // key of the k-th largest element
  const uint32_t ties = want;   // elements equal to it that are selected (the first ones by index)

  // ---- elements above / equal to the threshold in the slices before this one
  uint32_t gt_base = 0, eq_base = 0;
  if (n_ranks > 1) {
    if (tid < 2) slice_cnt[tid] = 0;
    __syncthreads();
    uint32_t g = 0, e = 0;
    for (int c0 = lo; c0 < hi; c0 += kStep) {
      const int i0 = c0 + tid * kTopkItems;
      uint32_t key[kTopkItems];
      topk_load8<T>(row, i0, hi, key);
#pragma unroll
      for (int j = 0; j < kTopkItems; ++j) {
        g += (i0 + j < hi && key[j] > thr) ? 1u : 0u;
        e += (i0 + j < hi && key[j] == thr) ? 1u : 0u;
      }
    }
    g = __reduce_add_sync(0xffffffffu, g);
    e = __reduce_add_sync(0xffffffffu, e);
    if (lane == 0) {
      atomicAdd(&slice_cnt[0], g);
      atomicAdd(&slice_cnt[1], e);
    }
    cluster.sync();
    for (int r = 0; r < rank; ++r) {
      const uint32_t* remote = cluster.map_shared_rank(slice_cnt, r);
      gt_base += remote[0];
      eq_base += remote[1];
    }
  }

  // ---- compaction in ascending index order
  for (int c0 = lo; c0 < hi; c0 += kStep) {
    const int i0 = c0 + tid * kTopkItems;
    uint32_t key[kTopkItems];
    topk_load8<T>(row, i0, hi, key);
    uint32_t g = 0, e = 0;
    bool isg[kTopkItems], ise[kTopkItems];
#pragma unroll
    for (int j = 0; j < kTopkItems; ++j) {
      isg[j] = i0 + j < hi && key[j] > thr;
      ise[j] = i0 + j < hi && key[j] == thr;
      g += isg[j];
      e += ise[j];
    }
    // block-wide exclusive scan of (g, e), packed into 16-bit halves (a step holds 8192 elements)
    const uint32_t v = g | (e << 16);
    uint32_t incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const uint32_t w = lane < kWarps ? warp_tot[lane] : 0u;
      uint32_t wi = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, wi, d);
        if (lane >= d) wi += up;
      }
      if (lane < kWarps) warp_tot[lane] = wi - w;  // exclusive
      if (lane == 31) chunk_tot = wi;
    }
    __syncthreads();
    const uint32_t excl = warp_tot[warp] + (incl - v);
    uint32_t g_before = gt_base + (excl & 0xffffu);
    uint32_t e_before = eq_base + (excl >> 16);
#pragma unroll
    for (int j = 0; j < kTopkItems; ++j) {
      if (isg[j] || (ise[j] && e_before < ties)) {
        const uint32_t pos = g_before + min(e_before, ties);
        out_idx[pos] = (IndexT)(i0 + j);
        if (out_val) out_val[pos] = row[i0 + j];
      }
      g_before += isg[j];
      e_before += ise[j];
    }
    const uint32_t tot = chunk_tot;
    gt_base += tot & 0xffffu;
    eq_base += tot >> 16;
    __syncthreads();  // warp_tot / chunk_tot are rewritten by the next step
  }
  cluster.sync();  // no CTA leaves while another may still read its shared memory
}

__device__ __forceinline__ float topk_to_float(float v) { return v; }
__device__ __forceinline__ float topk_to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float topk_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

// Threshold selection: per row the positions whose score is greater than `threshold`, in
// ascending order, and how many there are.  One CTA per row, one sweep, same block-wide scan as
// the compaction above.  `indices` holds n entries per row; those beyond the row's count are
// left untouched.
template <typename T, typename IndexT, int THREADS>
__global__ void __launch_bounds__(THREADS)
select_above_kernel(const T* __restrict__ scores, int n, float threshold, IndexT* __restrict__ indices,
                    int* __restrict__ counts) {
  constexpr int kTopkThreads = THREADS;  // shadows the namespace constant inside the kernel
  constexpr int kWarps = THREADS / 32;
  __shared__ uint32_t warp_tot[kTopkThreads / 32];
  __shared__ uint32_t chunk_tot;
  const T* row = scores + (size_t)blockIdx.x * n;
  IndexT* out_idx = indices + (size_t)blockIdx.x * n;
  const int tid = (int)threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int kStep = kTopkThreads * kTopkItems;
  uint32_t base = 0;
  for (int c0 = 0; c0 < n; c0 += kStep) {
    const int i0 = c0 + tid * kTopkItems;
    bool sel[kTopkItems];
    uint32_t g = 0;
#pragma unroll
    for (int j = 0; j < kTopkItems; ++j) {
      sel[j] = i0 + j < n && topk_to_float(row[i0 + j]) > threshold;
      g += sel[j];
    }
    uint32_t incl = g;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const uint32_t w = lane < kWarps ? warp_tot[lane] : 0u;
      uint32_t wi = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xffffffffu, wi, d);
        if (lane >= d) wi += up;
      }
      if (lane < kWarps) warp_tot[lane] = wi - w;  // exclusive
      if (lane == 31) chunk_tot = wi;
    }
    __syncthreads();
    uint32_t pos = base + warp_tot[warp] + (incl - g);
#pragma unroll
    for (int j = 0; j < kTopkItems; ++j) {
      if (sel[j]) out_idx[pos++] = (IndexT)(i0 + j);
    }
    base += chunk_tot;
    __syncthreads();  // warp_tot / chunk_tot are rewritten by the next step
  }
  if (tid == 0) counts[blockIdx.x] = (int)base;
}

}  // namespace fcr
