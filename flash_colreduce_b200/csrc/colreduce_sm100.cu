// flash_colreduce for B200 (sm_100a): device kernels and the C ABI in front of them.
//
// The operator is computed in two streaming passes that share one kernel
// template, each a warp-specialised persistent kernel:
//
//   rows pass  (PH_ROWS): a CTA keeps two 128-row Q tiles stationary in shared
//       memory and streams K tiles past them.  S = Q.K^T lands in tensor
//       memory with query rows on the 128 lanes, so each softmax thread owns
//       one query row and keeps its running max / sum in registers.  Output:
//       -log2-sum-exp2 of every row.
//   columns pass (PH_COLS): the operands swap roles.  A CTA keeps two 128-row
//       K tiles stationary and streams Q tiles, so S^T lands with key columns
//       on the lanes; each softmax thread owns one key column and folds
//       P = exp2(s*scale2 - lse_i) over the query dimension in a register.
//       No atomics and no cross-thread reduction; splits of the query range
//       go to a partial buffer that a last kernel combines in fixed order.
//
// Warp roles inside a CTA (608 threads, one CTA per SM): warps 0-15 are the
// softmax warps (two warpgroups of four warps per stationary tile, each folding
// every other accumulator tile of it), warp 16 issues the TMA loads and hands
// out work items, warps 17 and 18 issue tcgen05.mma (one per stationary tile;
// warp 17 also owns the tensor-memory allocation).  The columns pass of the max
// reduction has two more MMA warps (672 threads): one issuer per accumulator buffer.
//
// The arithmetic follows the reference kernel: scores are scaled by
// scale/ln(2) and exponentials are base 2 (flash_colreduce/flash.py:59-78,
// :108-124, :242, :291); masks follow flash.py:11-32; the causal tile ranges
// follow flash.py:201-207 but at 128-row granularity and with fully masked
// tiles never scheduled.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <array>
#include <atomic>
#include <mutex>
#include <string>
#include <type_traits>
#include <vector>

#include "plan.h"
#include "ptx_sm100.cuh"
#include "softmax_fold.cuh"

namespace fcr {

enum { PH_ROWS = 1, PH_COLS = 2 };

// Two softmax warpgroups per stationary sub-tile; they fold whole accumulator tiles in turn
// (warpgroup p folds the tiles that land in accumulator buffer p), independent of each other.
constexpr int kFoldGroups = 2;
constexpr int kSoftmaxWarps = 4 * kSubTiles * kFoldGroups;
constexpr int kProducerWarp = kSoftmaxWarps;
constexpr int kMmaWarp = kSoftmaxWarps + 1;   // issues the MMAs of sub-tile 0, owns the TMEM allocation
// MMA-issuing warps: one per stationary sub-tile, except in the columns pass of the max reduction,
// which has one per accumulator buffer (two per sub-tile).  That pass takes no exponentials, its
// folds are short, and with one issuer per sub-tile the tensor pipe waited for the issuer's barrier
// handshakes (8192-square, 128 heads: 1.17 -> 0.94 ms); the other passes are bound by the folds and
// lose to the extra warps' registers (measured 3-6 % slower), so they keep one issuer per sub-tile.
constexpr int kTmemCols = 512;
constexpr int kSpan = kTile;  // columns of an accumulator tile one thread folds: all of them
#ifndef FCR_CHUNK_ROWS
#define FCR_CHUNK_ROWS 64
#endif
#ifndef FCR_CHUNK_COLS
#define FCR_CHUNK_COLS 32
#endif
// accumulator columns per tensor-memory load: 64 in the rows pass (one running-max update
// per 64 keys), 32 in the columns pass (the lse operands cost registers)
constexpr int kChunkRows = FCR_CHUNK_ROWS;
constexpr int kChunkCols = FCR_CHUNK_COLS;
static_assert(kSpan % kChunkRows == 0 && kChunkRows % 32 == 0 && kSpan % kChunkCols == 0 &&
                  kChunkCols % 32 == 0, "chunk must divide the per-thread span");
constexpr long long kWaitLimitCycles = 2000000000LL;  // default bound of a device-side wait: about one second

// Device status codes (status word 0).  Word 1: block, word 2: thread, word 3: detail.
enum {
  ST_OK = 0,
  ST_SMEM_MISALIGNED = 1,
  ST_WAIT_STAT_EMPTY = 11,
  ST_WAIT_RING_EMPTY = 12,
  ST_WAIT_STAT_FULL = 21,
  ST_WAIT_RING_FULL = 22,
  ST_WAIT_TMEM_EMPTY = 23,
  ST_WAIT_DRAIN = 24,
  ST_WAIT_TMEM_FULL = 31,
  ST_WAIT_RING_FULL_SM = 32,
  ST_WAIT_LSE_EMPTY = 14,
  ST_WAIT_LSE_FULL = 27,
  ST_WAIT_SCHED_EMPTY = 13,
  ST_WAIT_SCHED_FULL = 26,
  ST_WAIT_SCHED_FULL_SM = 38,
  ST_WAIT_MERGE_FULL = 36,
  ST_WAIT_MERGE_EMPTY = 37,
};

struct PassParams : PassGeom {
  int m_pad, n_pad;
  float scale2;    // |scale| * log2(e)
  uint32_t idesc;  // tcgen05 instruction descriptor
  int tf32;        // fp32 operands multiplied as TF32 (else fp16 / bf16)
  int slab_elems;  // elements per 128-byte operand slab: 64 (16-bit) or 32 (fp32)
  float* neg_lse;  // [BH][m_pad]
  float* part_m;   // [n_split][BH][m_pad]
  float* part_l;   // [n_split][BH][m_pad]
  float* part_out; // [n_split][BH][n_pad]
  float* dump;     // [BH][M][n_pad] score cache of the key-streaming rows pass (null: none)
  void* out;       // [BH][N] of out_dtype
  int out_dtype;
  int mean_mode;   // 0: none, 1: divide by div_M, 2: causal rule
  int div_M, div_N, div_c;
  int* status;
  int* host_status;       // the device's status mailbox in mapped host memory (null: none)
  long long wait_limit;   // bound of every device-side wait, in clock64 cycles
  int skip_ring_load;     // self-test: CTA 0's TMA warp leaves out this ring load (-1: none)
  int* sched_counter;  // zero at launch; hands out work items beyond the first gridDim.x (null: round-robin)
  int clear_status;    // 1: this kernel clears status words 0-3 itself (no memset ran before it)
  int key_tiles;       // key-streaming kernels: 128-key tiles per head
  int fold_cols;       // key-streaming columns pass: M rounded up to a 32-query chunk
};

// First failure wins: the code goes to status word 0 of the workspace and, when the device has
// one, to the mailbox in mapped host memory, where the host sees it without a synchronisation.
__device__ __noinline__ void report_status(const PassParams& p, int code, int detail) {
  if (atomicCAS(p.status, 0, code) == 0) {
    p.status[1] = (int)blockIdx.x;
    p.status[2] = (int)threadIdx.x;
    p.status[3] = detail;
    if (p.host_status != nullptr) {
      volatile int* hs = p.host_status;
      hs[1] = (int)blockIdx.x;
      hs[2] = (int)threadIdx.x;
      hs[3] = detail;
      __threadfence_system();
      hs[0] = code;
    }
    __threadfence_system();
  }
}

// SHORT selects the buffering for work items that stream only a few tiles: two stationary
// stages, so that the next item's stationary tiles are fetched while this one is computed,
// at the price of a shallower streamed ring.  Long items keep one stationary stage and a
// deeper ring.
template <int DPAD, bool SHORT>
struct SmemLayout {
  static constexpr int kTileBytes = kTile * DPAD * 2;
  static constexpr int kHalves = DPAD / 64;     // 64-element (128-byte) column slabs per tile
  static constexpr int kHalfBytes = kTile * 128;
  // 512-byte rows (DPAD 256): the stationary block takes 128 KB, which leaves 64 KB for streaming.
  // A streamed tile then travels as two pieces of 256 bytes per row (two slabs), one ring slot
  // each, and the MMAs of a piece run while the next piece is loaded.
  static constexpr int kPieces = DPAD == 256 ? 2 : 1;        // ring slots per streamed tile
  static constexpr int kSlotBytes = kTileBytes / kPieces;    // bytes of a ring slot
  static constexpr int kSlotHalves = kHalves / kPieces;      // 128-byte slabs per ring slot
  static constexpr int KS = DPAD == 256 ? 1 : ((DPAD == 64 || SHORT) ? 2 : 1);  // stationary stages
  static constexpr int KR = DPAD == 256 ? 2 : (DPAD == 64 ? 6 : (SHORT ? 2 : 4));  // streamed ring slots
  static constexpr int kLseBytes = kTile * 4;
  // The lse values of a streamed query tile (columns pass) travel in a ring of their own, deeper
  // than the tile ring: the tile slots are then released by the MMAs alone and the loads run
  // ahead of the folds, which only hold the 512-byte lse slots.
  static constexpr int KL = KR + 4;  // tiles in the ring + tiles being folded + slack
  static constexpr int off_stat = 0;
  static constexpr int off_ring = off_stat + KS * kSubTiles * kTileBytes;
  static constexpr int off_lse = off_ring + KR * kSlotBytes;
  static constexpr int off_merge = off_lse + KL * kLseBytes;  // float2 [2 slots][kSubTiles][kTile]
  static constexpr int kMergeBytes = 2 * kSubTiles * kTile * 8;
  static constexpr int off_bars = off_merge + kMergeBytes;
  static constexpr int KI = 4;                   // work items announced ahead of their consumers
  static constexpr int kNumBars = 2 * KS + 2 * KR + 8 + 8 + 2 * KI + 2 * KL;
  static constexpr int off_misc = off_bars + 8 * kNumBars;
  static constexpr int kBytes = off_misc + 16 + 48 * KI;  // + the ring of announced work items
  static constexpr int kDynamicBytes = kBytes;
  static_assert(kDynamicBytes <= 232448, "exceeds the 227 KB shared memory of an sm_100 CTA");
};

// Bounded mbarrier wait.  Returns false when the wait limit expired here or in
// another thread of the CTA (the abort flag); the caller then leaves its loop.
// A failed mbarrier try_wait comes back after some tens of nanoseconds (whatever the suspend-time
// hint), so a waiting warp polls.  Letting the waiting warps sleep between polls was measured
// (100 ns to 1 us for the TMA and MMA warps, 50 and 200 ns for the fold warps): no timing changed by
// more than the run-to-run noise, so they simply poll.
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                         const PassParams& p, int code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++spins & 7u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > p.wait_limit) {
        *abort_flag = 1;
        report_status(p, code, (int)parity);
        return false;
      }
    }
  }
}
// Same, with a warp-uniform result so that .sync.aligned instructions that
// follow are executed by all 32 lanes or by none.
#define WAIT(bar, par, code) wait_bar_warp(bar, par, abort_flag, p, code)
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity,
                                              volatile int* abort_flag, const PassParams& p, int code) {
  const bool ok = wait_bar(bar, parity, abort_flag, p, code);
  return __all_sync(0xffffffffu, ok);
}

__device__ __forceinline__ float mean_divisor(const PassParams& p, int j) {
  if (p.mean_mode == 2 && j >= p.div_c) return (float)(p.div_N - j);
  return (float)p.div_M;
}

__device__ __forceinline__ void store_out(void* out, int out_dtype, size_t idx, float v) {
  if (out_dtype == FCR_F16) {
    reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
  } else if (out_dtype == FCR_BF16) {
    reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  } else {
    reinterpret_cast<float*>(out)[idx] = v;
  }
}

template <int PHASE, int RED>
__host__ __device__ constexpr bool mma_per_buffer() { return PHASE == PH_COLS && RED == RED_MAX; }
template <int PHASE, int RED>
__host__ __device__ constexpr int pass_threads() {
  return (kSoftmaxWarps + 1 + (mma_per_buffer<PHASE, RED>() ? 2 * kSubTiles : kSubTiles)) * 32;
}

template <int PHASE, int DPAD, int RED, bool SHORT>
__global__ void __launch_bounds__((pass_threads<PHASE, RED>()), 1)
pass_kernel(const __grid_constant__ CUtensorMap tmap_stat,
            const __grid_constant__ CUtensorMap tmap_strm, const PassParams p) {
  using L = SmemLayout<DPAD, SHORT>;
  constexpr int KS = L::KS, KR = L::KR;
  constexpr bool kMmaPerBuffer = mma_per_buffer<PHASE, RED>();
  constexpr int kMmaWarps = kMmaPerBuffer ? 2 * kSubTiles : kSubTiles;
  // The 128-byte swizzle of the operand tiles needs a 1024-byte aligned base;
  // the kernel uses no static shared memory, so the dynamic window starts there.
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = ptx::smem_u32(smem);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(p, ST_SMEM_MISALIGNED, (int)base);
    return;
  }

  const uint32_t s_stat = base + L::off_stat;
  const uint32_t s_ring = base + L::off_ring;
  const uint32_t s_lse = base + L::off_lse;
  const uint32_t bar0 = base + L::off_bars;
  auto bar_stat_full = [&](uint32_t ks) { return bar0 + 8u * ks; };
  auto bar_stat_empty = [&](uint32_t ks) { return bar0 + 8u * (KS + ks); };
  auto bar_ring_full = [&](uint32_t s) { return bar0 + 8u * (2 * KS + s); };
  auto bar_ring_empty = [&](uint32_t s) { return bar0 + 8u * (2 * KS + KR + s); };
  auto bar_tm_full = [&](uint32_t a, uint32_t ts) { return bar0 + 8u * (2 * KS + 2 * KR + a * 2 + ts); };
  auto bar_tm_empty = [&](uint32_t a, uint32_t ts) {
    return bar0 + 8u * (2 * KS + 2 * KR + 4 + a * 2 + ts);
  };
  auto bar_merge_full = [&](uint32_t a, uint32_t slot) {
    return bar0 + 8u * (2 * KS + 2 * KR + 8 + a * 2 + slot);
  };
  auto bar_merge_empty = [&](uint32_t a, uint32_t slot) {
    return bar0 + 8u * (2 * KS + 2 * KR + 12 + a * 2 + slot);
  };
  constexpr int KI = L::KI;
  auto bar_sched_full = [&](uint32_t i) { return bar0 + 8u * (2 * KS + 2 * KR + 16 + i); };
  auto bar_sched_empty = [&](uint32_t i) { return bar0 + 8u * (2 * KS + 2 * KR + 16 + KI + i); };
  constexpr int KL = L::KL;
  auto bar_lse_full = [&](uint32_t i) { return bar0 + 8u * (2 * KS + 2 * KR + 16 + 2 * KI + i); };
  auto bar_lse_empty = [&](uint32_t i) { return bar0 + 8u * (2 * KS + 2 * KR + 16 + 2 * KI + KL + i); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_misc + 4);
  // Announced work items, decoded once by the TMA warp (12 ints each; head -1 ends the kernel).
  volatile int* sched_ring = reinterpret_cast<volatile int*>(smem + L::off_misc + 16);
  auto read_item = [&](uint32_t slot) {
    const volatile int* e = sched_ring + slot * 12;
    Item g;
    g.bh = e[0];
    g.sp = e[1];
    g.c_lo = e[2];
    g.c_hi = e[3];
    g.par = e[10];
#pragma unroll
    for (int a = 0; a < kSubTiles; ++a) {
      g.r0[a] = e[4 + 3 * a];
      g.t_lo[a] = e[5 + 3 * a];
      g.t_hi[a] = e[6 + 3 * a];
    }
    return g;
  };

  const int warp = (int)(threadIdx.x >> 5);
  const int lane = (int)(threadIdx.x & 31);

  if (warp == 0) {  // the lanes of one warp initialise the barriers side by side
    if (lane < KS) {
      ptx::mbar_init(bar_stat_full(lane), 1);
      ptx::mbar_init(bar_stat_empty(lane), kMmaWarps);
    }
    if (lane < KR) {
      ptx::mbar_init(bar_ring_full(lane), 1);
      ptx::mbar_init(bar_ring_empty(lane), kMmaWarps);
    }
    if (lane < KL) {
      ptx::mbar_init(bar_lse_full(lane), 1);
      ptx::mbar_init(bar_lse_empty(lane), 4 * kSubTiles);
    }
    if (lane < 4) {
      const uint32_t a = (uint32_t)lane >> 1, ts = (uint32_t)lane & 1u;
      ptx::mbar_init(bar_tm_full(a, ts), 1);
      ptx::mbar_init(bar_tm_empty(a, ts), 4);
      ptx::mbar_init(bar_merge_full(a, ts), 4);
      ptx::mbar_init(bar_merge_empty(a, ts), 4);
    }
    if (lane < KI) {
      ptx::mbar_init(bar_sched_full(lane), 1);
      ptx::mbar_init(bar_sched_empty(lane), kMmaWarps + kSoftmaxWarps);
    }
    if (lane == 0) *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kProducerWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_stat);
    ptx::prefetch_tensormap(&tmap_strm);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Set-up is done: let the next kernel of the stream begin its own set-up as SMs free up,
  // and wait here for the previous kernel's results (the rows pass's lse, the work counters).
  if (threadIdx.x == 0) ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  if (p.clear_status && blockIdx.x == 0 && threadIdx.x < 4) p.status[threadIdx.x] = 0;

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------ TMA warp
    // Work items are handed out dynamically: the first is the CTA's own index,
    // later ones come from a global counter (fetched one item early, so that the
    // atomic's latency is hidden).  Each item is decoded here once and announced
    // to the other warps through a small ring in shared memory; head -1 ends the
    // kernel.  With two stationary stages the stationary tiles of item i+1 are
    // requested before the streamed tiles of item i, i.e. a whole item ahead.
    constexpr bool kAhead = KS >= 2;
    uint32_t ring_seq = 0, tile_seq = 0, item_seq = 0;  // ring slots, streamed tiles, items so far
    bool ok = true;
    auto load_stationary = [&](const Item& g, uint32_t seq) {
      const int b = g.bh / p.H, h = g.bh - b * p.H;
      const uint32_t ks = seq % KS, kph = (seq / KS) & 1u;
      if (!WAIT(bar_stat_empty(ks), kph ^ 1u, ST_WAIT_STAT_EMPTY)) return false;
      if (lane == 0) {
        ptx::mbar_arrive_expect_tx(bar_stat_full(ks), kSubTiles * L::kTileBytes);
#pragma unroll
        for (int a = 0; a < kSubTiles; ++a)
#pragma unroll
          for (int hf = 0; hf < L::kHalves; ++hf)
            ptx::tma_load_4d(s_stat + (ks * kSubTiles + a) * L::kTileBytes + hf * L::kHalfBytes,
                             &tmap_stat, bar_stat_full(ks), hf * p.slab_elems, g.r0[a], h, b);
      }
      __syncwarp();
      return true;
    };
    // Lane 0 asks the global counter for an index one item early and leaves the answer in
    // `pending`; it is broadcast only when the next iteration needs it, so the warp never
    // stalls on the atomic's round trip.
    int pending = 0;
    int dealt = (int)blockIdx.x;  // round-robin dealing: the item this CTA took last
    auto issue_fetch = [&]() {
      if (p.sched_counter == nullptr) {
        dealt += (int)gridDim.x;
        pending = dealt;
      } else if (lane == 0) {
        pending = (int)gridDim.x + atomicAdd(p.sched_counter, 1);
      }
    };
    const int item = (int)blockIdx.x;
    issue_fetch();
    Item g;
    g.bh = -1;
    if (item < p.n_items) g = decode_item<PHASE == PH_COLS>(p, item);
    if (kAhead && g.bh >= 0) ok = load_stationary(g, 0);
    for (; ok; ++item_seq) {
      const uint32_t si = item_seq % KI, sph = (item_seq / KI) & 1u;
      ok = WAIT(bar_sched_empty(si), sph ^ 1u, ST_WAIT_SCHED_EMPTY);
      if (!ok) break;
      const bool last = g.bh < 0;
      if (lane == 0) {
        volatile int* e = sched_ring + si * 12;
        e[0] = g.bh;
        if (!last) {
          e[1] = g.sp;
          e[2] = g.c_lo;
          e[3] = g.c_hi;
          e[10] = g.par;
#pragma unroll
          for (int a = 0; a < kSubTiles; ++a) {
            e[4 + 3 * a] = g.r0[a];
            e[5 + 3 * a] = g.t_lo[a];
            e[6 + 3 * a] = g.t_hi[a];
          }
        }
        ptx::mbar_arrive(bar_sched_full(si));
      }
      __syncwarp();
      if (last) break;
      // the item after this one (its index was requested an iteration ago), and a request
      // for the index of the one after that
      const int item_next = __shfl_sync(0xffffffffu, pending, 0);
      Item g_next;
      g_next.bh = -1;
      if (item_next < p.n_items) {
        g_next = decode_item<PHASE == PH_COLS>(p, item_next);
        issue_fetch();
      }
      if (kAhead) {
        if (g_next.bh >= 0) ok = load_stationary(g_next, item_seq + 1);
      } else {
        ok = load_stationary(g, item_seq);
      }
      if (!ok) break;
      const int b = g.bh / p.H, h = g.bh - b * p.H;
      for (int t = g.c_lo; t < g.c_hi; ++t, ++tile_seq) {
#pragma unroll
        for (int piece = 0; piece < L::kPieces; ++piece, ++ring_seq) {
          const uint32_t s = ring_seq % KR, ph = (ring_seq / KR) & 1u;
          ok = WAIT(bar_ring_empty(s), ph ^ 1u, ST_WAIT_RING_EMPTY);
          if (!ok) break;
          // self-test of the bounded waits: one load of CTA 0 is never requested (nothing is in
          // flight for its slot), so the consumers' waits on it run into their limit
          const bool left_out = blockIdx.x == 0 && (int)ring_seq == p.skip_ring_load;
          if (lane == 0 && !left_out) {
            ptx::mbar_arrive_expect_tx(bar_ring_full(s), L::kSlotBytes);
#pragma unroll
            for (int hf = 0; hf < L::kSlotHalves; ++hf)
              ptx::tma_load_4d(s_ring + s * L::kSlotBytes + hf * L::kHalfBytes, &tmap_strm,
                               bar_ring_full(s), (piece * L::kSlotHalves + hf) * p.slab_elems,
                               t * kTile, h, b);
          }
          __syncwarp();
        }
        if (!ok) break;
        if (PHASE == PH_COLS) {  // the tile's lse values, into their own ring
          const uint32_t sl = tile_seq % KL, lph = (tile_seq / KL) & 1u;
          ok = WAIT(bar_lse_empty(sl), lph ^ 1u, ST_WAIT_LSE_EMPTY);
          if (!ok) break;
          if (lane == 0) {
            ptx::mbar_arrive_expect_tx(bar_lse_full(sl), L::kLseBytes);
            ptx::bulk_load(s_lse + sl * L::kLseBytes,
                           p.neg_lse + (size_t)g.bh * p.m_pad + (size_t)t * kTile, L::kLseBytes,
                           bar_lse_full(sl));
          }
          __syncwarp();
        }
      }
      g = g_next;
    }
  } else if (warp >= kMmaWarp) {
    // ----------------------------------------------------------- MMA warps
    // One issuing warp per stationary sub-tile (per accumulator buffer in the max columns pass):
    // tcgen05.mma issue blocks while the tensor pipe's short queue is full, so with a single
    // issuer the pipe drains during that warp's barrier handshakes; with several, one warp's
    // handshakes overlap another's MMAs.
    const int a = (warp - kMmaWarp) % kSubTiles;
    const int my_buf = (warp - kMmaWarp) / kSubTiles;  // non-zero only with one issuer per accumulator buffer
    // Accumulator buffer of a tile = (its index within the work item + the item's parity) mod 2,
    // so that the warpgroup that folds it does not depend on which items this CTA happened to get;
    // tm_use[b] counts the uses of buffer b and gives its barrier phase.
    uint32_t ring_seq = 0, item_seq = 0, tile_seq = 0;
    uint32_t tm_use[2] = {0, 0};
    bool ok = true;
    for (;; ++item_seq) {
      const uint32_t si = item_seq % KI, sph = (item_seq / KI) & 1u;
      ok = WAIT(bar_sched_full(si), sph, ST_WAIT_SCHED_FULL);
      if (!ok) break;
      const Item g = read_item(si);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_sched_empty(si));
      if (g.bh < 0) break;
      const uint32_t ks = item_seq % KS, kph = (item_seq / KS) & 1u;
      ok = WAIT(bar_stat_full(ks), kph, ST_WAIT_STAT_FULL);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t a_addr = s_stat + (ks * kSubTiles + a) * L::kTileBytes;
      for (int t = g.c_lo; ok && t < g.c_hi; ++t, ++tile_seq) {
        const uint32_t ts = (uint32_t)(t - g.t_lo[a] + g.par) & 1u;
        const bool in_range = t >= g.t_lo[a] && t < g.t_hi[a];
        const bool my_tile = in_range && (!kMmaPerBuffer || (int)ts == my_buf);
        if (PHASE == PH_COLS) {
          // The softmax warps read a tile's lse values from the lse ring once its product is in
          // tensor memory, without waiting on the lse barrier themselves: this warp waits for the
          // values before it issues the tile's MMAs, so a completed product implies they have
          // landed.  An lse slot is released by eight arrivals, four per sub-tile: the four warps
          // that fold the tile for the sub-tile, or, when the tile is outside the sub-tile's range,
          // this warp on their behalf -- after its own wait, so that the arrivals of a use of the
          // slot can never reach the barrier before the use before it has completed.
          const uint32_t sl = tile_seq % KL, lph = (tile_seq / KL) & 1u;
          ok = WAIT(bar_lse_full(sl), lph, ST_WAIT_LSE_FULL);
          if (!ok) break;
          if (!in_range && my_buf == 0) {
            if (lane == 0) ptx::mbar_arrive_count(bar_lse_empty(sl), 4);
            __syncwarp();
          }
        }
        // a streamed tile arrives in kPieces ring slots (one, or two halves of the row width)
#pragma unroll
        for (int piece = 0; piece < L::kPieces; ++piece, ++ring_seq) {
          const uint32_t s = ring_seq % KR, ph = (ring_seq / KR) & 1u;
          ok = WAIT(bar_ring_full(s), ph, ST_WAIT_RING_FULL);
          if (!ok) break;
          if (my_tile) {
            if (piece == 0) {
              const uint32_t tph = (ts ? tm_use[1] : tm_use[0]) & 1u;
              ok = WAIT(bar_tm_empty(a, ts), tph ^ 1u, ST_WAIT_TMEM_EMPTY);
              if (!ok) break;
            }
            ptx::tc_fence_after_sync();
            if (lane == 0) {
              const uint32_t d = tmem_base + (uint32_t)(a * 2 + ts) * kTile;
              const uint32_t b_addr = s_ring + s * L::kSlotBytes;
              // One instruction per 32 bytes of each operand row: 16 halves or 8 TF32 values.
              // The operand kind is chosen once, outside the unrolled sequence.
              constexpr int kSteps = DPAD / 16 / L::kPieces;  // instructions per ring slot
              auto issue_steps = [&](auto as_tf32) {
#pragma unroll
                for (int kq = 0; kq < kSteps; ++kq) {
                  const int kk = piece * kSteps + kq;  // step within the whole row
                  const uint32_t a_off = (uint32_t)(kk >> 2) * L::kHalfBytes + (uint32_t)(kk & 3) * 32u;
                  const uint32_t b_off = (uint32_t)(kq >> 2) * L::kHalfBytes + (uint32_t)(kq & 3) * 32u;
                  if constexpr (decltype(as_tf32)::value)
                    ptx::umma_tf32(d, ptx::smem_desc_sw128(a_addr + a_off),
                                   ptx::smem_desc_sw128(b_addr + b_off), p.idesc, kk > 0 ? 1u : 0u);
                  else
                    ptx::umma_f16(d, ptx::smem_desc_sw128(a_addr + a_off),
                                  ptx::smem_desc_sw128(b_addr + b_off), p.idesc, kk > 0 ? 1u : 0u);
                }
              };
              if (p.tf32)
                issue_steps(std::true_type{});
              else
                issue_steps(std::false_type{});
              if (piece + 1 == L::kPieces) ptx::umma_commit(bar_tm_full(a, ts));
              ptx::umma_commit(bar_ring_empty(s));
            }
            __syncwarp();
            if (piece + 1 == L::kPieces) {
              if (ts) ++tm_use[1]; else ++tm_use[0];
            }
          } else {
            // not this sub-tile's tile: the slot is released as soon as it has been filled
            if (lane == 0) ptx::mbar_arrive(bar_ring_empty(s));
            __syncwarp();
          }
        }
      }
      if (!ok) break;
      if (lane == 0) ptx::umma_commit(bar_stat_empty(ks));
      __syncwarp();
    }
    if (ok && item_seq > 0) {
      // The last commit covers every MMA issued: wait for it so that no
      // asynchronous arrive is still outstanding when the CTA retires.
      const uint32_t last = item_seq - 1;
      WAIT(bar_stat_empty(last % KS), (last / KS) & 1u, ST_WAIT_DRAIN);
    }
  } else {
    // -------------------------------------------------------- softmax warps
    // Warp w reads tensor-memory lanes 32*(w%4).. (a hardware rule), belongs to
    // stationary sub-tile a and to fold group `part` of it: it folds the accumulator
    // tiles of sub-tile a that land in buffer `part`, all 128 columns of each.
    const int a = (warp >> 2) % kSubTiles;
    const int part = warp / (4 * kSubTiles);
    const int tid_wg = (warp & 3) * 32 + lane;
    const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
    float2* merge_buf = reinterpret_cast<float2*>(smem + L::off_merge);
    uint32_t ring_base = 0, merge_seq = 0;
    uint32_t tm_use = 0;  // uses of accumulator buffer (a, part) so far: gives its barrier phase
    const uint32_t taddr = tmem_base + lane_field + (uint32_t)(a * 2 + part) * kTile;
    bool ok = true;
    for (uint32_t item_seq = 0;; ++item_seq) {
      const uint32_t si = item_seq % KI, sph = (item_seq / KI) & 1u;
      ok = WAIT(bar_sched_full(si), sph, ST_WAIT_SCHED_FULL_SM);
      if (!ok) break;
      const Item g = read_item(si);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(bar_sched_empty(si));
      if (g.bh < 0) break;
      const int mine = g.r0[a] + tid_wg;  // query row (rows pass) or key column (columns pass)
      float m_run = -INFINITY, l_run = 0.f;
      float acc[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = (RED == RED_MAX) ? -INFINITY : 0.f;
      // Per item: the streamed indices this thread's row / column may use, [valid_lo, valid_hi),
      // and which tiles intersect a mask edge (all others take the unmasked code path).
      int valid_lo = 0, valid_hi, mask_from, mask_until = 0;
      if (PHASE == PH_COLS) {
        // queries i with max(mine - off, 0) <= i < M attend key `mine`
        valid_lo = p.causal ? max(mine - p.off, 0) : 0;
        valid_hi = p.M;
        mask_from = p.M >> 7;  // the ragged last tile, if any
        mask_until = p.causal ? max(g.r0[a] + 2 * kTile - 2 - p.off, 0) >> 7 : 0;  // diagonal tiles
      } else {
        // keys j <= min(N - 1, mine + off) are attended by query `mine`
        valid_hi = p.causal ? (int)min((long long)p.N, (long long)mine + p.off + 1) : p.N;
        mask_from = p.N >> 7;
        if (p.causal) mask_from = (int)min((long long)mask_from, ((long long)g.r0[a] + p.off + 1) >> 7);
      }

      // Tile t of the item goes to accumulator buffer (t - t_lo[a] + par) mod 2: it alternates
      // within the item, starting from the parity of the item's index (a property of the item,
      // so the summation order does not depend on which CTA runs it, and short items spread
      // over both fold groups).  This group folds every other tile of the sub-tile's range.
      for (int t = g.t_lo[a] + ((part - g.par) & 1); t < g.t_hi[a]; t += 2) {
        const uint32_t tph = tm_use & 1u;
        ++tm_use;
        ok = WAIT(bar_tm_full(a, part), tph, ST_WAIT_TMEM_FULL);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const int c0 = t * kTile;  // streamed index of the tile's first column
        const bool need_mask = t >= mask_from || t < mask_until;
        const int lim_lo = valid_lo - c0, lim_hi = valid_hi - c0;
        // columns pass: the tile's lse values, in the lse ring slot of the tile's running number
        // (they have landed: the MMA warp waited for them before it issued the tile's MMAs)
        const uint32_t sl = (ring_base + (uint32_t)(t - g.c_lo)) % KL;
        const float* lse_s = reinterpret_cast<const float*>(smem + L::off_lse + sl * L::kLseBytes);

        constexpr int kChunk = (PHASE == PH_COLS) ? kChunkCols : kChunkRows;
        uint32_t ra[kChunk];
        // one chunk at a time: the other warps of the scheduler cover the load latency
#pragma unroll
        for (int c = 0; c < kSpan / kChunk; ++c) {
          ptx::tmem_ld<kChunk>(taddr + c * kChunk, ra);
          ptx::tmem_ld_wait<kChunk>(ra);
          if (c + 1 == kSpan / kChunk) {
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_tm_empty(a, part));
          }
          if constexpr (PHASE == PH_ROWS) {
            if (need_mask)
              rows_chunk<true, kChunk>(ra, p.scale2, lim_hi - kChunk * c, m_run, l_run);
            else
              rows_chunk<false, kChunk>(ra, p.scale2, kChunk, m_run, l_run);
          } else {
            if (need_mask)
              cols_chunk<RED, true, kChunk>(ra, lse_s + kChunk * c, p.scale2, lim_lo - kChunk * c,
                                            lim_hi - kChunk * c, acc);
            else
              cols_chunk<RED, false, kChunk>(ra, lse_s + kChunk * c, p.scale2, 0, kChunk, acc);
          }
        }
        if (PHASE == PH_COLS) {
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_lse_empty(sl));
        }
      }
      ring_base += (uint32_t)(g.c_hi - g.c_lo);
      if (!ok) break;
      if (g.r0[a] >= p.LS) continue;  // nothing to write for this sub-tile

      // ------------------------------------------------------ item epilogue
      // The two threads that share a row / column (one per fold group) combine their
      // partial state through shared memory; the thread of group 0 writes the result.
      float v0, v1 = 0.f;
      if (PHASE == PH_ROWS) {
        v0 = m_run;
        v1 = l_run;
      } else if (RED == RED_SUM) {
        v0 = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      } else {
        v0 = fmaxf(fmaxf(acc[0], acc[1]), fmaxf(acc[2], acc[3]));
      }
      {
        const uint32_t slot = merge_seq & 1u, mph = (merge_seq >> 1) & 1u;
        float2* cell = merge_buf + ((size_t)slot * kSubTiles + a) * kTile + tid_wg;
        ++merge_seq;
        if (part != 0) {
          ok = WAIT(bar_merge_empty(a, slot), mph ^ 1u, ST_WAIT_MERGE_EMPTY);
          if (!ok) break;
          *cell = make_float2(v0, v1);
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_merge_full(a, slot));
          continue;
        }
        ok = WAIT(bar_merge_full(a, slot), mph, ST_WAIT_MERGE_FULL);
        if (!ok) break;
        const float2 other = *cell;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_merge_empty(a, slot));
        if (PHASE == PH_ROWS) {
          const float mx = fmaxf(v0, other.x);
          const float ms = (mx == -INFINITY) ? 0.f : mx;
          v1 = v1 * ptx::ex2(v0 - ms) + other.y * ptx::ex2(other.x - ms);
          v0 = mx;
        } else if (RED == RED_SUM) {
          v0 += other.x;
        } else {
          v0 = fmaxf(v0, other.x);
        }
      }
      if (PHASE == PH_ROWS) {
        if (mine < p.M) {
          if (p.n_split == 1) {
            p.neg_lse[(size_t)g.bh * p.m_pad + mine] = -(v0 + log2f(v1));
          } else {
            const size_t idx = ((size_t)g.sp * p.BH + g.bh) * p.m_pad + mine;
            p.part_m[idx] = v0;
            p.part_l[idx] = v1;
          }
        }
      } else if (PHASE == PH_COLS) {
        if (mine < p.N) {
          float v = (RED == RED_SUM) ? v0 : ptx::ex2(v0);
          if (p.n_split == 1) {
            if (p.mean_mode) v = v / mean_divisor(p, mine);
            store_out(p.out, p.out_dtype, (size_t)g.bh * p.N + mine, v);
          } else {
            p.part_out[((size_t)g.sp * p.BH + g.bh) * p.n_pad + mine] = v;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------- teardown
  __syncwarp();
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // A wait expired somewhere: give loads that may still be in flight time to
    // land in this CTA's shared memory before it is released.
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fcr
#include "keystream_sm100.cuh"
#include "topk.cuh"
namespace fcr {

// Combines the per-split running (max, sum) of the rows pass into -lse.
__global__ void combine_lse_kernel(const float* __restrict__ part_m,
                                   const float* __restrict__ part_l, float* __restrict__ neg_lse,
                                   int n_split, size_t per_split, int m_pad, int M) {
  ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  const size_t total = per_split;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % m_pad);
    if (i >= M) continue;
    float mx = -INFINITY;
    for (int s = 0; s < n_split; ++s) mx = fmaxf(mx, part_m[s * per_split + idx]);
    float l = 0.f;
    for (int s = 0; s < n_split; ++s) {
      const float ms = part_m[s * per_split + idx];
      if (ms != -INFINITY) l = fmaf(part_l[s * per_split + idx], exp2f(ms - mx), l);
    }
    neg_lse[idx] = -(mx + log2f(l));
  }
}

// Combines the per-split column partials in split order, applies the mean
// divisor and casts (flash_colreduce/flash.py:308, :377-385).
__global__ void final_reduce_kernel(const float* __restrict__ part, PassParams p, int is_max) {
  ptx::grid_dependency_wait();
  const size_t per_split = (size_t)p.BH * p.n_pad;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < per_split;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int j = (int)(idx % p.n_pad);
    if (j >= p.N) continue;
    const size_t bh = idx / p.n_pad;
    float v = part[idx];
    for (int s = 1; s < p.n_split; ++s) {
      const float w = part[s * per_split + idx];
      v = is_max ? fmaxf(v, w) : v + w;
    }
    if (p.mean_mode) v = v / mean_divisor(p, j);
    store_out(p.out, p.out_dtype, bh * p.N + j, v);
  }
}

// Columns pass from cached scores (decode with M <= 16): thread = key column, the M raw scores of
// the column are read from the array the rows pass wrote, P = 2^(s*scale2 - lse_i) is folded in
// query order (flash_colreduce/flash.py:120-124), then the mean divisor and the cast (:377-385).
template <int RED>
__global__ void __launch_bounds__(256)
scores_reduce_kernel(const float* __restrict__ scores, PassParams p, int blocks_per_head) {
  __shared__ float nl[16];
  ptx::grid_dependency_wait();
  const int bh = (int)(blockIdx.x / (unsigned)blocks_per_head);
  // four consecutive keys per thread: one 16-byte load per query row
  const int j0 = ((int)(blockIdx.x % (unsigned)blocks_per_head) * 256 + (int)threadIdx.x) * 4;
  if ((int)threadIdx.x < p.M) nl[threadIdx.x] = p.neg_lse[(size_t)bh * p.m_pad + threadIdx.x];
  __syncthreads();
  if (j0 >= p.N) return;
  const float* col = scores + (size_t)bh * p.M * p.n_pad + j0;  // n_pad is a multiple of 128: aligned
  float acc[4];
  int lo[4];  // queries lo <= i < M attend key j
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    acc[e] = (RED == RED_MAX) ? -INFINITY : 0.f;
    lo[e] = p.causal ? max(j0 + e - p.off, 0) : 0;
  }
  for (int i = lo[0]; i < p.M; ++i) {  // lo[0] is the smallest of the four
    const float4 s4 = *reinterpret_cast<const float4*>(col + (size_t)i * p.n_pad);
    const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x = fmaf(sv[e], p.scale2, nl[i]);
      if (RED == RED_MAX)
        acc[e] = (i >= lo[e]) ? fmaxf(acc[e], x) : acc[e];
      else
        acc[e] += (i >= lo[e]) ? ptx::ex2(x) : 0.f;
    }
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if (j0 + e >= p.N) break;
    float v = (RED == RED_MAX) ? ptx::ex2(acc[e]) : acc[e];
    if (p.mean_mode) v = v / mean_divisor(p, j0 + e);
    store_out(p.out, p.out_dtype, (size_t)bh * p.N + j0 + e, v);
  }
}

// Mean divisor + cast of an already reduced fp32 (B*H, N) array.
__global__ void finalize_kernel(const float* __restrict__ acc, PassParams p) {
  const size_t total = (size_t)p.BH * p.N;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int j = (int)(idx % p.N);
    float v = acc[idx];
    if (p.mean_mode) v = v / mean_divisor(p, j);
    store_out(p.out, p.out_dtype, idx, v);
  }
}

// ===================================================================== host
static thread_local std::string g_last_error;

// Per-thread trace: CUDA events recorded around the two passes of each call.
struct Trace {
  bool on = false;
  int used = 0;
  std::vector<std::array<cudaEvent_t, 3>> events;
};
static thread_local Trace g_trace;

static cudaEvent_t trace_event(int which) {
  if (!g_trace.on) return nullptr;
  if (which == 0) {
    if (g_trace.used >= 256) return nullptr;
    if ((int)g_trace.events.size() <= g_trace.used) {
      std::array<cudaEvent_t, 3> e{};
      for (auto& ev : e)
        if (cudaEventCreate(&ev) != cudaSuccess) return nullptr;
      g_trace.events.push_back(e);
    }
  }
  if (g_trace.used >= (int)g_trace.events.size()) return nullptr;
  return g_trace.events[g_trace.used][which];
}
static void trace_mark(int which, cudaStream_t stream) {
  cudaEvent_t ev = trace_event(which);
  if (ev) cudaEventRecord(ev, stream);
  if (ev && which == 2) ++g_trace.used;
}

static int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}
static int cuda_fail(cudaError_t e, const char* what) {
  return fail(FCR_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// Tensor map over a (B,H,rows,D) tensor viewed as 4-D (D, rows, H, B); a box
// is 64 elements x 128 rows of one head, written to shared memory with the
// 128-byte swizzle.  Elements beyond D or beyond `rows` read as zero.
static int make_tensor_map(CUtensorMap* map, const void* ptr, int dtype, int D, int rows, int H,
                           int B, const int64_t* strides) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return fail(FCR_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0)
    return fail(FCR_ERR_UNSUPPORTED, "q / k base address must be 16-byte aligned");
  const int elem_bytes = dtype == FCR_F32 ? 4 : 2;
  const int align_elems = 16 / elem_bytes;
  const int64_t fallback = align_up64((int64_t)D, align_elems);
  auto stride_bytes = [&](int dim, int64_t s) -> cuuint64_t {
    if (dim <= 1 && (s <= 0 || s % align_elems != 0)) s = fallback;  // never dereferenced
    return (cuuint64_t)s * (cuuint64_t)elem_bytes;
  };
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t gstr[3] = {stride_bytes(rows, strides[2]), stride_bytes(H, strides[1]),
                        stride_bytes(B, strides[0])};
  cuuint32_t box[4] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)kTile, 1u, 1u};  // 128-byte slab
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  const CUtensorMapDataType dt = dtype == FCR_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == FCR_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 4, const_cast<void*>(ptr), dims, gstr, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(FCR_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
  return FCR_OK;
}

// Facts about a device and the resources the library keeps on it, looked up once per device.
struct DeviceInfo {
  bool ready = false;
  int index = 0;
  int sms = 0;
  // Status mailbox: 16 ints of pinned host memory mapped into the device's address space.  A
  // kernel whose bounded wait expires writes its status there as well as into the workspace, so
  // the next library call on the device sees the failure without synchronising anything.
  int* mailbox_host = nullptr;
  int* mailbox_dev = nullptr;
};
static std::mutex g_dev_mutex;
static DeviceInfo g_dev[64];

// The current device's entry.  With `want_mailbox` the mailbox is allocated on first use (the
// only allocation the library ever makes: 64 bytes of pinned host memory per device).
static int device_info(const DeviceInfo** out, bool want_mailbox) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(FCR_ERR_UNSUPPORTED, "device ordinal beyond 63");
  DeviceInfo& d = g_dev[dev];
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!d.ready) {
    int major = 0, sms = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
    if (major != 10)
      return fail(FCR_ERR_UNSUPPORTED,
                  "this library contains sm_100a code only; the current device has compute capability major " +
                      std::to_string(major));
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
    d.index = dev;
    d.sms = sms;
    d.ready = true;
  }
  if (want_mailbox && !d.mailbox_host) {
    void* h = nullptr;
    void* dptr = nullptr;
    e = cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable);
    if (e != cudaSuccess) return cuda_fail(e, "cudaHostAlloc(status mailbox)");
    memset(h, 0, 64);
    e = cudaHostGetDevicePointer(&dptr, h, 0);
    if (e != cudaSuccess) {
      cudaFreeHost(h);
      return cuda_fail(e, "cudaHostGetDevicePointer(status mailbox)");
    }
    d.mailbox_dev = reinterpret_cast<int*>(dptr);
    d.mailbox_host = reinterpret_cast<int*>(h);
  }
  *out = &d;
  return FCR_OK;
}

static int device_sm_count(int* out) {
  const DeviceInfo* d = nullptr;
  const int rc = device_info(&d, false);
  if (rc != FCR_OK) return rc;
  *out = d->sms;
  return FCR_OK;
}

static std::string status_text(const volatile int* w) {
  return "device status " + std::to_string(w[0]) + " (block " + std::to_string(w[1]) + ", thread " +
         std::to_string(w[2]) + ", detail " + std::to_string(w[3]) + "): a bounded wait inside a kernel expired";
}

// A failure a kernel left in the device's mailbox is reported once, by the first library call
// that looks; the mailbox is then cleared.
static int check_mailbox(const DeviceInfo& d, int32_t* code_out) {
  if (code_out) *code_out = 0;
  volatile int* w = d.mailbox_host;
  if (!w || w[0] == 0) return FCR_OK;
  if (code_out) *code_out = w[0];
  const std::string msg = status_text(w) + " in an earlier call on this device; its output is not valid";
  w[0] = 0;
  return fail(FCR_ERR_DEVICE_TIMEOUT, msg);
}

// Kernel launches made by the library in this process.
static std::atomic<long long> g_launches{0};

// Overrides for the self-test of the bounded waits (calling thread only).
static thread_local long long g_wait_limit_override = 0;
static thread_local int g_skip_ring_load = -1;

static uint32_t instr_desc(int dtype, bool negate_a) {
  // kind::f16 / kind::tf32, fp32 accumulate, both operands K-major, M = 128, N = 128
  const uint32_t fmt = dtype == FCR_F32 ? 2u : (dtype == FCR_BF16 ? 1u : 0u);
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((negate_a ? 1u : 0u) << 13) |
         ((uint32_t)(kTile >> 3) << 17) | ((uint32_t)(kTile >> 4) << 24);
}

// Launches `kern`; with `dependent` it may begin while the previous kernel of the stream is
// still running (the kernels call grid_dependency_wait() before reading its results).
template <typename... KArgs, typename... Args>
static cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, bool dependent, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent ? 1 : 0;
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Device the calling thread's current operator call runs on (set by run_colreduce).
static thread_local int t_device = 0;

template <int PHASE, int DPAD, int RED, bool SHORT>
static int launch_pass(const CUtensorMap& stat, const CUtensorMap& strm, const PassParams& pp,
                       int ctas, cudaStream_t stream) {
  auto kern = pass_kernel<PHASE, DPAD, RED, SHORT>;
  constexpr int smem = SmemLayout<DPAD, SHORT>::kDynamicBytes;
  // the shared-memory opt-in is per kernel and device: do it once for each
  static std::atomic<unsigned long long> opted_in{0};
  cudaError_t e = cudaSuccess;
  const unsigned long long bit = 1ULL << (t_device & 63);
  if (!(opted_in.load(std::memory_order_acquire) & bit)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
    opted_in.fetch_or(bit, std::memory_order_release);
  }
  // Every pass kernel may begin its set-up while the kernel before it in the stream drains (they all
  // wait for that kernel's completion before touching global memory): the columns pass follows the rows
  // pass or its combine kernel, the rows pass the previous call's last kernel.
  e = launch_kernel(kern, dim3(ctas), dim3(pass_threads<PHASE, RED>()), smem, stream, true, stat, strm, pp);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "pass kernel launch");
  return FCR_OK;
}

template <int PHASE, int RED>
static int launch_pass_d(int d_pad, bool short_items, const CUtensorMap& stat,
                         const CUtensorMap& strm, const PassParams& pp, int ctas,
                         cudaStream_t stream) {
  if (d_pad == 64) return launch_pass<PHASE, 64, RED, false>(stat, strm, pp, ctas, stream);
  if (d_pad == 256) return launch_pass<PHASE, 256, RED, false>(stat, strm, pp, ctas, stream);
  if (short_items) return launch_pass<PHASE, 128, RED, true>(stat, strm, pp, ctas, stream);
  return launch_pass<PHASE, 128, RED, false>(stat, strm, pp, ctas, stream);
}

template <int PHASE, int DPAD, int RED>
static int launch_keystream(const CUtensorMap& map_q, const CUtensorMap& map_k, const PassParams& pp,
                            int ctas, cudaStream_t stream) {
  auto kern = keystream_kernel<PHASE, DPAD, RED>;
  constexpr int smem = KeyStreamSmem<DPAD>::kDynamicBytes;
  static std::atomic<unsigned long long> opted_in{0};
  cudaError_t e = cudaSuccess;
  const unsigned long long bit = 1ULL << (t_device & 63);
  if (!(opted_in.load(std::memory_order_acquire) & bit)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
    opted_in.fetch_or(bit, std::memory_order_release);
  }
  e = launch_kernel(kern, dim3(ctas), dim3(kKsThreads), smem, stream, true, map_q, map_k, pp);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "key-streaming kernel launch");
  return FCR_OK;
}

template <int PHASE, int RED>
static int launch_keystream_d(int d_pad, const CUtensorMap& map_q, const CUtensorMap& map_k,
                              const PassParams& pp, int ctas, cudaStream_t stream) {
  if (d_pad == 64) return launch_keystream<PHASE, 64, RED>(map_q, map_k, pp, ctas, stream);
  if (d_pad == 256) return launch_keystream<PHASE, 256, RED>(map_q, map_k, pp, ctas, stream);
  return launch_keystream<PHASE, 128, RED>(map_q, map_k, pp, ctas, stream);
}

// Bytes a plan cannot do without: the score cache is the last region of the workspace and is
// optional (without it the columns pass sweeps K a second time).
static int64_t min_workspace_bytes(const fcr_plan& pl) {
  return pl.score_cache ? pl.off_scores : pl.workspace_bytes;
}

static int check_workspace(const fcr_plan& pl, const void* ws, size_t ws_bytes) {
  if (!ws) return fail(FCR_ERR_WORKSPACE, "workspace is null");
  if ((reinterpret_cast<uintptr_t>(ws) & 255u) != 0)
    return fail(FCR_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  if ((int64_t)ws_bytes < min_workspace_bytes(pl))
    return fail(FCR_ERR_WORKSPACE, "workspace of " + std::to_string(ws_bytes) +
                                       " bytes is smaller than the required " +
                                       std::to_string(min_workspace_bytes(pl)));
  return FCR_OK;
}

static void fill_common(PassParams& pp, const fcr_problem& pr, const fcr_plan& pl, uint8_t* ws,
                        bool cols, int* host_status) {
  memset(&pp, 0, sizeof(pp));
  static_cast<PassGeom&>(pp) = pass_geometry(pr, pl, cols);
  pp.m_pad = pl.m_pad;
  pp.n_pad = pl.n_pad;
  float s2 = fabsf(pr.scale) * 1.4426950408889634f;
  if (!(s2 >= 1e-30f)) s2 = 1e-30f;  // scale 0: every score becomes (numerically) zero
  pp.scale2 = s2;
  pp.idesc = instr_desc(pr.in_dtype, pr.scale < 0.f);
  pp.tf32 = pr.in_dtype == FCR_F32 ? 1 : 0;
  pp.slab_elems = pr.in_dtype == FCR_F32 ? 32 : 64;
  pp.neg_lse = reinterpret_cast<float*>(ws + pl.off_neg_lse);
  pp.part_m = reinterpret_cast<float*>(ws + pl.off_part_m);
  pp.part_l = reinterpret_cast<float*>(ws + pl.off_part_l);
  pp.part_out = reinterpret_cast<float*>(ws + pl.off_part_out);
  pp.status = reinterpret_cast<int*>(ws + pl.off_status);
  pp.sched_counter = pl.static_schedule ? nullptr : pp.status + (cols ? 9 : 8);
  pp.clear_status = (pl.static_schedule && !cols) ? 1 : 0;  // the first kernel of a call that ran no memset
  pp.host_status = host_status;
  pp.wait_limit = g_wait_limit_override > 0 ? g_wait_limit_override : kWaitLimitCycles;
  pp.skip_ring_load = g_skip_ring_load;
}

static void fill_mean(PassParams& pp, int reduction, int is_causal, int M, int N) {
  pp.div_M = M;
  pp.div_N = N;
  pp.div_c = N > M ? N - M : 0;
  pp.mean_mode = reduction == FCR_MEAN ? (is_causal ? 2 : 1) : 0;
}

// CTAs per row: one when the rows alone fill the GPU, else a cluster of 2, 4 or 8 that splits the
// row, as long as every CTA keeps at least one full sweep step (8192 elements).
static int topk_cluster_size(int rows, int n, int sms) {
  int c = 1;
  while (c < 8 && (long long)rows * c * 2 <= sms && n / (c * 2) >= kTopkThreads * kTopkItems) c *= 2;
  return c;
}

template <typename T, typename IndexT>
static int launch_topk_t(const void* scores, int rows, int n, int k, void* indices, void* values,
                         int cluster, int small_rows_from, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)rows * cluster);
  cfg.blockDim = dim3(kTopkThreads);
  cfg.stream = stream;  // both launch shapes below go to the caller's stream
  // many short rows: 256-thread blocks, several rows per SM at a time
  const bool small = cluster == 1 && n <= 16 * kTopkThreadsSmall * kTopkItems && rows >= small_rows_from;
  if (small) {
    cfg.blockDim = dim3(kTopkThreadsSmall);
    cfg.numAttrs = 0;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t es = cudaLaunchKernelEx(&cfg, topk_kernel<T, IndexT, kTopkThreadsSmall, 8>,
                                        static_cast<const T*>(scores), n, k, static_cast<IndexT*>(indices),
                                        static_cast<T*>(values));
    if (es == cudaSuccess) es = cudaGetLastError();
    if (es != cudaSuccess) return cuda_fail(es, "topk launch");
    return FCR_OK;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster > 1 ? 1 : 0;  // a single CTA per row is an ordinary launch
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaLaunchKernelEx(&cfg, topk_kernel<T, IndexT, kTopkThreads, 32>, static_cast<const T*>(scores), n, k,
                                     static_cast<IndexT*>(indices), static_cast<T*>(values));
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "topk launch");
  return FCR_OK;
}

template <typename T>
static int launch_topk(const void* scores, int rows, int n, int k, void* indices, int index_bits,
                       void* values, cudaStream_t stream) {
  int sms = 0;
  const int rc = device_sm_count(&sms);
  if (rc != FCR_OK) return rc;
  const int cluster = topk_cluster_size(rows, n, sms);
  if (index_bits == 64)
    return launch_topk_t<T, long long>(scores, rows, n, k, indices, values, cluster, 2 * sms, stream);
  return launch_topk_t<T, int>(scores, rows, n, k, indices, values, cluster, 2 * sms, stream);
}

template <typename T, typename IndexT>
static void launch_select_t(const void* scores, int rows, int n, float threshold, void* indices, int* counts,
                            bool small, cudaStream_t stream) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (small)
    select_above_kernel<T, IndexT, kTopkThreadsSmall><<<rows, kTopkThreadsSmall, 0, stream>>>(
        static_cast<const T*>(scores), n, threshold, static_cast<IndexT*>(indices), counts);
  else
    select_above_kernel<T, IndexT, kTopkThreads><<<rows, kTopkThreads, 0, stream>>>(
        static_cast<const T*>(scores), n, threshold, static_cast<IndexT*>(indices), counts);
}

template <typename T>
static int launch_select(const void* scores, int rows, int n, float threshold, void* indices,
                         int index_bits, int* counts, cudaStream_t stream) {
  int sms = 0;
  const int rc = device_sm_count(&sms);
  if (rc != FCR_OK) return rc;
  // many short rows: 256-thread blocks, several rows per SM at a time (as for the top-k)
  const bool small = n <= 16 * kTopkThreadsSmall * kTopkItems && rows >= 2 * sms;
  if (index_bits == 64)
    launch_select_t<T, long long>(scores, rows, n, threshold, indices, counts, small, stream);
  else
    launch_select_t<T, int>(scores, rows, n, threshold, indices, counts, small, stream);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "select_above launch");
  return FCR_OK;
}

}  // namespace fcr

using namespace fcr;

extern "C" {

const char* fcr_version(void) { return "0.1.0"; }

const char* fcr_last_error(void) { return g_last_error.c_str(); }

int fcr_plan_problem(const fcr_problem* problem, int32_t num_sms, fcr_plan* plan) {
  if (!problem || !plan) return fail(FCR_ERR_BAD_ARG, "null problem or plan");
  int sms = num_sms;
  if (sms <= 0) {
    const int rc = device_sm_count(&sms);
    if (rc != FCR_OK) return rc;
  }
  std::string err;
  const int rc = plan_problem(*problem, sms, *plan, err);
  if (rc != FCR_OK) return fail(rc, err);
  return FCR_OK;
}

int fcr_plan_item(const fcr_problem* problem, const fcr_plan* plan, int32_t pass, int32_t item,
                  int32_t* out) {
  if (!problem || !plan || !out) return fail(FCR_ERR_BAD_ARG, "null argument");
  if (pass != 1 && pass != 2) return fail(FCR_ERR_BAD_ARG, "pass must be 1 (rows) or 2 (columns)");
  const PassGeom g = pass_geometry(*problem, *plan, pass == 2);
  if (item < 0 || item >= g.n_items) return fail(FCR_ERR_BAD_ARG, "item out of range");
  if (plan->key_stream) {
    int bh, sp, t_lo, t_hi;
    keystream_item(plan->key_chunks, plan->n_pad / kTile, item, bh, sp, t_lo, t_hi);
    const int32_t v[10] = {bh, sp, t_lo, t_hi, 0, t_lo, t_hi, plan->m_pad, t_lo, t_lo};
    memcpy(out, v, sizeof(v));
    return FCR_OK;
  }
  const Item it = pass == 2 ? decode_item<true>(g, item) : decode_item<false>(g, item);
  out[0] = it.bh;
  out[1] = it.sp;
  out[2] = it.c_lo;
  out[3] = it.c_hi;
  for (int a = 0; a < kSubTiles; ++a) {
    out[4 + 3 * a] = it.r0[a];
    out[5 + 3 * a] = it.t_lo[a];
    out[6 + 3 * a] = it.t_hi[a];
  }
  return FCR_OK;
}

size_t fcr_workspace_bytes(const fcr_problem* problem, int32_t num_sms) {
  fcr_plan pl;
  if (fcr_plan_problem(problem, num_sms, &pl) != FCR_OK) return 0;
  return (size_t)pl.workspace_bytes;
}

}  // extern "C"

// Plans of the calling thread's recent problems: a repeat call with the same problem struct on
// the same device plans nothing (the plan depends on the problem and the SM count only).
struct PlanCacheEntry {
  fcr_problem problem;
  int device;
  fcr_plan plan;
};
static bool same_problem(const fcr_problem& a, const fcr_problem& b) {
  return a.B == b.B && a.H == b.H && a.M == b.M && a.N == b.N && a.D == b.D &&
         memcmp(a.q_strides, b.q_strides, sizeof(a.q_strides)) == 0 &&
         memcmp(a.k_strides, b.k_strides, sizeof(a.k_strides)) == 0 && a.in_dtype == b.in_dtype &&
         a.reduction == b.reduction && a.is_causal == b.is_causal &&
         memcmp(&a.scale, &b.scale, sizeof(float)) == 0 && a.causal_offset == b.causal_offset &&
         a.mean_M == b.mean_M && a.mean_N == b.mean_N;
}
static int plan_for_call(const fcr_problem& pr, const DeviceInfo& dev, const fcr_plan** out) {
  constexpr int kEntries = 8;
  static thread_local PlanCacheEntry cache[kEntries];
  static thread_local int used = 0, next = 0;
  for (int i = 0; i < used; ++i)
    if (cache[i].device == dev.index && same_problem(cache[i].problem, pr)) {
      *out = &cache[i].plan;
      return FCR_OK;
    }
  std::string err;
  fcr_plan pl;
  const int rc = plan_problem(pr, dev.sms, pl, err);
  if (rc != FCR_OK) return fail(rc, err);
  PlanCacheEntry& e = cache[next];
  e.problem = pr;
  e.device = dev.index;
  e.plan = pl;
  *out = &e.plan;
  next = (next + 1) % kEntries;
  if (used < kEntries) ++used;
  return FCR_OK;
}

// The operator proper, behind fcr_colreduce and fcr_colreduce_static.
static int run_colreduce(const fcr_problem& pr, const fcr_plan& pl, const DeviceInfo& dev, const void* q,
                         const void* k, void* out, int32_t out_dtype, void* workspace,
                         size_t workspace_bytes, cudaStream_t stream) {
  int rc = check_workspace(pl, workspace, workspace_bytes);
  if (rc != FCR_OK) return rc;
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  t_device = dev.index;
  int* const mailbox = dev.mailbox_dev;

  CUtensorMap map_q, map_k;
  rc = make_tensor_map(&map_q, q, pr.in_dtype, pr.D, pr.M, pr.H, pr.B, pr.q_strides);
  if (rc != FCR_OK) return rc;
  rc = make_tensor_map(&map_k, k, pr.in_dtype, pr.D, pr.N, pr.H, pr.B, pr.k_strides);
  if (rc != FCR_OK) return rc;

  // Plans that draw work items from a counter clear it (and the status words) here; the others
  // clear their four status words in the first kernel and save this stream operation.
  cudaError_t e = cudaSuccess;
  if (!pl.static_schedule) {
    e = cudaMemsetAsync(ws + pl.off_status, 0, kStatusWords * 4, stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync");
  }

  if (pl.key_stream) {
    // Decode shapes: both passes stream the key tiles past the head's one query tile.
    trace_mark(0, stream);
    PassParams pp;
    auto fill = [&](bool cols) {
      fill_common(pp, pr, pl, ws, cols, mailbox);
      pp.n_split = pl.key_chunks;
      pp.n_items = pl.row_items;
      pp.key_tiles = pl.n_pad / kTile;
      pp.fold_cols = (int)align_up64(pr.M, kChunkCols);
    };
    fill(false);
    // the score cache is used when the caller's workspace has room for it
    const bool use_cache = pl.score_cache && (int64_t)workspace_bytes >= pl.workspace_bytes;
    if (use_cache) pp.dump = reinterpret_cast<float*>(ws + pl.off_scores);
    rc = launch_keystream_d<PH_ROWS, RED_SUM>(pl.d_pad, map_q, map_k, pp, pl.row_ctas, stream);
    if (rc != FCR_OK) return rc;
    {
      const size_t per_split = (size_t)pp.BH * pl.m_pad;
      const int blocks = (int)std::min<size_t>((per_split + 255) / 256, 4096);
      e = launch_kernel(combine_lse_kernel, dim3(blocks), dim3(256), 0, stream, true, pp.part_m,
                        pp.part_l, pp.neg_lse, pl.row_splits, per_split, pl.m_pad, pr.M);
      if (e == cudaSuccess) e = cudaGetLastError();
      if (e != cudaSuccess) return cuda_fail(e, "combine_lse launch");
    }
    trace_mark(1, stream);
    fill(true);
    pp.out = out;
    pp.out_dtype = out_dtype;
    fill_mean(pp, pr.reduction, pr.is_causal, pr.mean_M > 0 ? pr.mean_M : pr.M,
              pr.mean_N > 0 ? pr.mean_N : pr.N);
    if (use_cache) {
      const float* scores = reinterpret_cast<const float*>(ws + pl.off_scores);
      const int bph = (pr.N + 1023) / 1024;  // 256 threads x 4 keys
      const long long blocks = (long long)pp.BH * bph;
      if (blocks > 0x7fffffffLL) return fail(FCR_ERR_UNSUPPORTED, "problem has too many key blocks");
      if (pr.reduction == FCR_MAX)
        e = launch_kernel(scores_reduce_kernel<RED_MAX>, dim3((unsigned)blocks), dim3(256), 0, stream, true,
                          scores, pp, bph);
      else
        e = launch_kernel(scores_reduce_kernel<RED_SUM>, dim3((unsigned)blocks), dim3(256), 0, stream, true,
                          scores, pp, bph);
      if (e == cudaSuccess) e = cudaGetLastError();
      if (e != cudaSuccess) return cuda_fail(e, "scores_reduce launch");
      trace_mark(2, stream);
      return FCR_OK;
    }
    if (pr.reduction == FCR_MAX)
      rc = launch_keystream_d<PH_COLS, RED_MAX>(pl.d_pad, map_q, map_k, pp, pl.col_ctas, stream);
    else
      rc = launch_keystream_d<PH_COLS, RED_SUM>(pl.d_pad, map_q, map_k, pp, pl.col_ctas, stream);
    if (rc != FCR_OK) return rc;
    trace_mark(2, stream);
    return FCR_OK;
  }

  // rows pass: Q stationary, K streamed
  trace_mark(0, stream);
  PassParams pp;
  fill_common(pp, pr, pl, ws, false, mailbox);
  rc = launch_pass_d<PH_ROWS, RED_SUM>(pl.d_pad, (pl.short_items & 1) != 0, map_q, map_k, pp,
                                       pl.row_ctas, stream);
  if (rc != FCR_OK) return rc;
  if (pl.row_splits > 1) {
    const size_t per_split = (size_t)pp.BH * pl.m_pad;
    const int blocks = (int)std::min<size_t>((per_split + 255) / 256, 4096);
    e = launch_kernel(combine_lse_kernel, dim3(blocks), dim3(256), 0, stream, true, pp.part_m,
                      pp.part_l, pp.neg_lse, pl.row_splits, per_split, pl.m_pad, pr.M);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "combine_lse launch");
  }

  // columns pass: K stationary, Q streamed
  trace_mark(1, stream);
  fill_common(pp, pr, pl, ws, true, mailbox);
  pp.out = out;
  pp.out_dtype = out_dtype;
  fill_mean(pp, pr.reduction, pr.is_causal, pr.mean_M > 0 ? pr.mean_M : pr.M,
            pr.mean_N > 0 ? pr.mean_N : pr.N);
  if (pr.reduction == FCR_MAX)
    rc = launch_pass_d<PH_COLS, RED_MAX>(pl.d_pad, (pl.short_items & 2) != 0, map_k, map_q, pp,
                                         pl.col_ctas, stream);
  else
    rc = launch_pass_d<PH_COLS, RED_SUM>(pl.d_pad, (pl.short_items & 2) != 0, map_k, map_q, pp,
                                         pl.col_ctas, stream);
  if (rc != FCR_OK) return rc;
  if (pl.col_splits > 1) {
    const size_t per_split = (size_t)pp.BH * pl.n_pad;
    const int blocks = (int)std::min<size_t>((per_split + 255) / 256, 4096);
    e = launch_kernel(final_reduce_kernel, dim3(blocks), dim3(256), 0, stream, true, pp.part_out, pp,
                      (int)(pr.reduction == FCR_MAX));
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "final_reduce launch");
  }
  trace_mark(2, stream);
  return FCR_OK;
}

extern "C" {

int fcr_colreduce(const fcr_problem* problem, const void* q, const void* k, void* out,
                  int32_t out_dtype, void* workspace, size_t workspace_bytes, void* stream_v) {
  if (!problem || !q || !k || !out) return fail(FCR_ERR_BAD_ARG, "null argument");
  if (out_dtype != FCR_F16 && out_dtype != FCR_BF16 && out_dtype != FCR_F32)
    return fail(FCR_ERR_BAD_ARG, "invalid out_dtype");
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev, true);
  if (rc != FCR_OK) return rc;
  rc = check_mailbox(*dev, nullptr);  // a wait that expired in an earlier call is reported here
  if (rc != FCR_OK) return rc;
  const fcr_plan* pl = nullptr;
  rc = plan_for_call(*problem, *dev, &pl);
  if (rc != FCR_OK) return rc;
  return run_colreduce(*problem, *pl, *dev, q, k, out, out_dtype, workspace, workspace_bytes,
                       reinterpret_cast<cudaStream_t>(stream_v));
}

int64_t fcr_launch_count(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

int fcr_poll_device_status(int32_t* code_out) {
  const DeviceInfo* dev = nullptr;
  const int rc = device_info(&dev, false);
  if (rc != FCR_OK) return rc;
  return check_mailbox(*dev, code_out);
}

int fcr_self_test_hooks(int64_t wait_limit_cycles, int32_t skip_ring_load) {
  if (wait_limit_cycles < 0) return fail(FCR_ERR_BAD_ARG, "wait_limit_cycles must not be negative");
  g_wait_limit_override = wait_limit_cycles;
  g_skip_ring_load = skip_ring_load < 0 ? -1 : skip_ring_load;
  return FCR_OK;
}

int fcr_trace_enable(int32_t on) {
  g_trace.on = on != 0;
  g_trace.used = 0;
  return FCR_OK;
}

int32_t fcr_trace_count(void) { return g_trace.used; }

int fcr_trace_read(int32_t index, float* rows_ms, float* cols_ms) {
  if (index < 0 || index >= g_trace.used || !rows_ms || !cols_ms)
    return fail(FCR_ERR_BAD_ARG, "trace index out of range or null output");
  auto& e = g_trace.events[index];
  cudaError_t err = cudaEventSynchronize(e[2]);
  if (err != cudaSuccess) return cuda_fail(err, "cudaEventSynchronize");
  err = cudaEventElapsedTime(rows_ms, e[0], e[1]);
  if (err != cudaSuccess) return cuda_fail(err, "cudaEventElapsedTime");
  err = cudaEventElapsedTime(cols_ms, e[1], e[2]);
  if (err != cudaSuccess) return cuda_fail(err, "cudaEventElapsedTime");
  return FCR_OK;
}

int fcr_finalize(const float* acc, void* out, int32_t out_dtype, int32_t B, int32_t H, int32_t M,
                 int32_t N, int32_t reduction, int32_t is_causal, void* stream_v) {
  if (!acc || !out || B <= 0 || H <= 0 || M <= 0 || N <= 0)
    return fail(FCR_ERR_BAD_ARG, "null pointer or non-positive size");
  if (out_dtype != FCR_F16 && out_dtype != FCR_BF16 && out_dtype != FCR_F32)
    return fail(FCR_ERR_BAD_ARG, "invalid out_dtype");
  if (reduction != FCR_SUM && reduction != FCR_MEAN && reduction != FCR_MAX)
    return fail(FCR_ERR_BAD_ARG, "invalid reduction code");
  PassParams pp;
  memset(&pp, 0, sizeof(pp));
  pp.BH = B * H;
  pp.N = N;
  pp.M = M;
  pp.out = out;
  pp.out_dtype = out_dtype;
  fill_mean(pp, reduction, is_causal, M, N);
  const size_t total = (size_t)pp.BH * N;
  const int blocks = (int)std::min<size_t>((total + 255) / 256, 4096);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  finalize_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_v)>>>(acc, pp);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "finalize launch");
  return FCR_OK;
}

// Synchronises `stream`, then reads the four leading status words at `status_dev`.
static int read_status_words(const void* status_dev, cudaStream_t stream, int32_t* code_out) {
  int32_t words[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyAsync(words, status_dev, sizeof(words), cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(status)");
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
  if (code_out) *code_out = words[0];
  if (words[0] == ST_OK) return FCR_OK;
  // the same failure also sits in the device's mailbox: it is reported here, once
  const DeviceInfo* dev = nullptr;
  if (device_info(&dev, false) == FCR_OK && dev->mailbox_host) {
    volatile int* w = dev->mailbox_host;
    if (w[0] == words[0] && w[1] == words[1] && w[2] == words[2]) w[0] = 0;
  }
  return fail(FCR_ERR_DEVICE_TIMEOUT, status_text(words));
}

int fcr_read_device_status(const void* workspace, void* stream_v, int32_t* code_out) {
  if (!workspace) return fail(FCR_ERR_BAD_ARG, "null workspace");
  return read_status_words(workspace, reinterpret_cast<cudaStream_t>(stream_v), code_out);
}

// ----------------------------------------------------------------------
// Operator for callers that may not allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc: a plugin running
// inside another runtime's enqueue hook (the runtime owns every byte of the
// device and forbids allocation there), a serving loop that reserved its whole
// memory budget up front, or code that must not touch an allocator because the
// surrounding framework's caching allocator is locked or not reachable from C.
// For them the workspace fcr_colreduce needs lives in the library image
// itself: a fixed array in device global memory, present on every GPU that
// loads the library for as long as the process runs.
constexpr size_t kStaticScratchBytes = FCR_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the symbol, not a
// device address, so the address is looked up once per device (with that
// device current) and remembered.
static std::mutex g_scratch_mutex;
static void* g_scratch_addr[64] = {};

static int static_scratch_address(int dev, void** out) {
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    if (!ptr) return fail(FCR_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return FCR_OK;
}

int fcr_colreduce_static(const fcr_problem* problem, const void* q, const void* k, void* out,
                         int32_t out_dtype, void* stream_v) {
  if (!problem || !q || !k || !out) return fail(FCR_ERR_BAD_ARG, "null argument");
  if (out_dtype != FCR_F16 && out_dtype != FCR_BF16 && out_dtype != FCR_F32)
    return fail(FCR_ERR_BAD_ARG, "invalid out_dtype");
  // No mailbox is created here (that would be an allocation); one that fcr_colreduce created
  // earlier on this device is used and checked like there.
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev, false);
  if (rc != FCR_OK) return rc;
  rc = check_mailbox(*dev, nullptr);
  if (rc != FCR_OK) return rc;
  const fcr_plan* pl = nullptr;
  rc = plan_for_call(*problem, *dev, &pl);
  if (rc != FCR_OK) return rc;
  if ((size_t)min_workspace_bytes(*pl) > kStaticScratchBytes)
    return fail(FCR_ERR_WORKSPACE,
                "this problem needs " + std::to_string(min_workspace_bytes(*pl)) +
                    " bytes of scratch but the built-in scratch holds " +
                    std::to_string(kStaticScratchBytes) +
                    " (FCR_STATIC_SCRATCH_BYTES); use fcr_colreduce with a caller-owned workspace");
  void* scratch = nullptr;
  rc = static_scratch_address(dev->index, &scratch);
  if (rc != FCR_OK) return rc;
  // Same kernels as fcr_colreduce, handed the built-in array.  The status words
  // and scheduler counters at its start are cleared on the stream by that call;
  // everything else in the array is written before it is read.
  return run_colreduce(*problem, *pl, *dev, q, k, out, out_dtype, scratch, kStaticScratchBytes,
                       reinterpret_cast<cudaStream_t>(stream_v));
}

int fcr_read_device_status_static(void* stream_v, int32_t* code_out) {
  const DeviceInfo* dev = nullptr;
  int rc = device_info(&dev, false);
  if (rc != FCR_OK) return rc;
  void* scratch = nullptr;
  rc = static_scratch_address(dev->index, &scratch);
  if (rc != FCR_OK) return rc;
  return read_status_words(scratch, reinterpret_cast<cudaStream_t>(stream_v), code_out);
}

int fcr_topk(const void* scores, int32_t dtype, int32_t rows, int32_t n, int32_t k, void* indices,
             int32_t index_bits, void* values, void* stream_v) {
  if (!scores || !indices) return fail(FCR_ERR_BAD_ARG, "null scores or indices");
  if (rows <= 0 || n <= 0) return fail(FCR_ERR_BAD_ARG, "rows and n must be positive");
  if (k < 1 || k > n)
    return fail(FCR_ERR_BAD_ARG, "k = " + std::to_string(k) + " must lie in [1, n = " + std::to_string(n) + "]");
  if (index_bits != 32 && index_bits != 64) return fail(FCR_ERR_BAD_ARG, "index_bits must be 32 or 64");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  switch (dtype) {
    case FCR_F16: return launch_topk<__half>(scores, rows, n, k, indices, index_bits, values, stream);
    case FCR_BF16: return launch_topk<__nv_bfloat16>(scores, rows, n, k, indices, index_bits, values, stream);
    case FCR_F32: return launch_topk<float>(scores, rows, n, k, indices, index_bits, values, stream);
    default: return fail(FCR_ERR_BAD_ARG, "invalid dtype");
  }
}

int fcr_select_above(const void* scores, int32_t dtype, int32_t rows, int32_t n, float threshold,
                     void* indices, int32_t index_bits, int32_t* counts, void* stream_v) {
  if (!scores || !indices || !counts) return fail(FCR_ERR_BAD_ARG, "null scores, indices or counts");
  if (rows <= 0 || n <= 0) return fail(FCR_ERR_BAD_ARG, "rows and n must be positive");
  if (index_bits != 32 && index_bits != 64) return fail(FCR_ERR_BAD_ARG, "index_bits must be 32 or 64");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  switch (dtype) {
    case FCR_F16: return launch_select<__half>(scores, rows, n, threshold, indices, index_bits, counts, stream);
    case FCR_BF16:
      return launch_select<__nv_bfloat16>(scores, rows, n, threshold, indices, index_bits, counts, stream);
    case FCR_F32: return launch_select<float>(scores, rows, n, threshold, indices, index_bits, counts, stream);
    default: return fail(FCR_ERR_BAD_ARG, "invalid dtype");
  }
}

}  // extern "C"

#include "sharded.cuh"
