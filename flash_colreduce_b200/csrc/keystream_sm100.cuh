// Key-streaming kernels for the decode shapes: all M <= 128 queries of a head
// fit one tile, the keys are long.  Both passes keep the query tile of the
// current head in shared memory and stream that head's key tiles through a deep
// ring whose slots are released as soon as the MMAs that read them have retired,
// so that the loads run ahead of the softmax warps by the depth of the ring.
//
//   rows pass     S = Q K^T, lanes = queries: thread owns a query row and folds
//                 every fourth key tile of the work item into (max, sum); the four
//                 warpgroups leave four partial states, combined by
//                 combine_lse_kernel (flash_colreduce/flash.py:71-78).  With at most
//                 16 queries it also stores the raw scores (PassParams::dump), from
//                 which scores_reduce_kernel reduces the columns without a second
//                 sweep over the keys.
//   columns pass  S^T = K Q^T, lanes = keys: thread owns a key column; one tile
//                 holds every query, so the column's reduction is complete after
//                 one tile and is written straight to the output
//                 (flash_colreduce/flash.py:120-124, :377-385).
//
// Included by colreduce_sm100.cu after the shared helpers (PassParams, WAIT,
// store_out, mean_divisor).
#pragma once

namespace fcr {

constexpr int kKsSoftmaxWarps = 16;  // four warpgroups, one per accumulator buffer
constexpr int kKsProducerWarp = kKsSoftmaxWarps;
constexpr int kKsMmaWarp = kKsSoftmaxWarps + 1;
constexpr int kKsThreads = (kKsSoftmaxWarps + 2) * 32;
constexpr int kKsBuffers = 4;  // accumulator tiles in tensor memory: 4 x 128 columns

enum {
  ST_KS_WAIT_Q_EMPTY = 51,
  ST_KS_WAIT_RING_EMPTY = 52,
  ST_KS_WAIT_Q_FULL = 53,
  ST_KS_WAIT_RING_FULL = 54,
  ST_KS_WAIT_TMEM_EMPTY = 55,
  ST_KS_WAIT_DRAIN = 56,
  ST_KS_WAIT_TMEM_FULL = 57,
  ST_KS_WAIT_Q_FULL_SM = 58,
};

template <int DPAD>
struct KeyStreamSmem {
  static constexpr int kTileBytes = kTile * DPAD * 2;
  static constexpr int kHalves = DPAD / 64;
  static constexpr int kHalfBytes = kTile * 128;
  static constexpr int KR = DPAD == 64 ? 8 : (DPAD == 128 ? 5 : 2);  // key tiles in flight
  static constexpr int kLseBytes = kTile * 4;
  static constexpr int off_q = 0;
  static constexpr int off_ring = off_q + kTileBytes;
  static constexpr int off_lse = off_ring + KR * kTileBytes;
  static constexpr int off_bars = off_lse + kLseBytes;
  static constexpr int kNumBars = 2 + 2 * KR + 2 * kKsBuffers;
  static constexpr int off_misc = off_bars + 8 * kNumBars;
  static constexpr int kDynamicBytes = off_misc + 16;
  static_assert(kDynamicBytes <= 232448, "exceeds the 227 KB shared memory of an sm_100 CTA");
};

template <int PHASE, int DPAD, int RED>
__global__ void __launch_bounds__(kKsThreads, 1)
keystream_kernel(const __grid_constant__ CUtensorMap tmap_q,
                 const __grid_constant__ CUtensorMap tmap_k, const PassParams p) {
  static_assert(PHASE == PH_ROWS || PHASE == PH_COLS, "rows or columns pass");
  using L = KeyStreamSmem<DPAD>;
  constexpr int KR = L::KR;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = ptx::smem_u32(smem);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(p, ST_SMEM_MISALIGNED, (int)base);
    return;
  }
  const uint32_t s_q = base + L::off_q;
  const uint32_t s_ring = base + L::off_ring;
  const uint32_t s_lse = base + L::off_lse;
  const uint32_t bar0 = base + L::off_bars;
  const uint32_t bar_q_full = bar0, bar_q_empty = bar0 + 8u;
  auto bar_ring_full = [&](uint32_t s) { return bar0 + 8u * (2 + s); };
  auto bar_ring_empty = [&](uint32_t s) { return bar0 + 8u * (2 + KR + s); };
  auto bar_tm_full = [&](uint32_t b) { return bar0 + 8u * (2 + 2 * KR + b); };
  auto bar_tm_empty = [&](uint32_t b) { return bar0 + 8u * (2 + 2 * KR + kKsBuffers + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::off_misc + 4);

  const int warp = (int)(threadIdx.x >> 5);
  const int lane = (int)(threadIdx.x & 31);

  if (threadIdx.x == 0) {
    ptx::mbar_init(bar_q_full, 1);
    // the query tile (and, in the columns pass, the lse values beside it) is released by the
    // MMA warp's commit and by every softmax warp that read the lse values
    ptx::mbar_init(bar_q_empty, PHASE == PH_COLS ? 1 + kKsSoftmaxWarps : 1);
    for (int i = 0; i < KR; ++i) {
      ptx::mbar_init(bar_ring_full(i), 1);
      ptx::mbar_init(bar_ring_empty(i), 1);
    }
    for (int b = 0; b < kKsBuffers; ++b) {
      ptx::mbar_init(bar_tm_full(b), 1);
      ptx::mbar_init(bar_tm_empty(b), 4);
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == kKsMmaWarp) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    ptx::tmem_relinquish();
  }
  if (warp == kKsProducerWarp && lane == 0) {
    ptx::prefetch_tensormap(&tmap_q);
    ptx::prefetch_tensormap(&tmap_k);
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  if (p.clear_status && blockIdx.x == 0 && threadIdx.x < 4) p.status[threadIdx.x] = 0;

  // CTA c runs the contiguous items [c*I/G, (c+1)*I/G): consecutive items mostly belong to
  // one head, whose query tile is then loaded once.  Every warp derives the sequence itself.
  const int S = p.n_split;
  const int item_lo = (int)(((long long)p.n_items * blockIdx.x) / gridDim.x);
  const int item_hi = (int)(((long long)p.n_items * (blockIdx.x + 1)) / gridDim.x);

  if (warp == kKsProducerWarp) {
    // ------------------------------------------------------------ TMA warp
    uint32_t ring_seq = 0, q_seq = 0;
    int cur_bh = -1;
    bool ok = true;
    for (int item = item_lo; ok && item < item_hi; ++item) {
      int bh, sp, t_lo, t_hi;
      keystream_item(S, p.key_tiles, item, bh, sp, t_lo, t_hi);
      const int b = bh / p.H, h = bh - b * p.H;
      if (bh != cur_bh) {
        ok = WAIT(bar_q_empty, (q_seq & 1u) ^ 1u, ST_KS_WAIT_Q_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(bar_q_full,
                                     L::kTileBytes + (PHASE == PH_COLS ? L::kLseBytes : 0));
#pragma unroll
          for (int hf = 0; hf < L::kHalves; ++hf)
            ptx::tma_load_4d(s_q + hf * L::kHalfBytes, &tmap_q, bar_q_full, hf * p.slab_elems, 0, h, b);
          if (PHASE == PH_COLS)
            ptx::bulk_load(s_lse, p.neg_lse + (size_t)bh * p.m_pad, L::kLseBytes, bar_q_full);
        }
        __syncwarp();
        ++q_seq;
        cur_bh = bh;
      }
      for (int t = t_lo; t < t_hi; ++t, ++ring_seq) {
        const uint32_t s = ring_seq % KR, ph = (ring_seq / KR) & 1u;
        ok = WAIT(bar_ring_empty(s), ph ^ 1u, ST_KS_WAIT_RING_EMPTY);
        if (!ok) break;
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(bar_ring_full(s), L::kTileBytes);
#pragma unroll
          for (int hf = 0; hf < L::kHalves; ++hf)
            ptx::tma_load_4d(s_ring + s * L::kTileBytes + hf * L::kHalfBytes, &tmap_k,
                             bar_ring_full(s), hf * p.slab_elems, t * kTile, h, b);
        }
        __syncwarp();
      }
    }
  } else if (warp == kKsMmaWarp) {
    // ------------------------------------------------------------- MMA warp
    uint32_t ring_seq = 0, q_seq = 0;
    uint32_t tm_par = 0;  // bit b: parity of the next use of accumulator buffer b
    int cur_bh = -1;
    bool ok = true;
    for (int item = item_lo; ok && item < item_hi; ++item) {
      int bh, sp, t_lo, t_hi;
      keystream_item(S, p.key_tiles, item, bh, sp, t_lo, t_hi);
      if (bh != cur_bh) {
        ok = WAIT(bar_q_full, q_seq & 1u, ST_KS_WAIT_Q_FULL);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        ++q_seq;
        cur_bh = bh;
      }
      for (int t = t_lo; t < t_hi; ++t, ++ring_seq) {
        const uint32_t s = ring_seq % KR, ph = (ring_seq / KR) & 1u;
        ok = WAIT(bar_ring_full(s), ph, ST_KS_WAIT_RING_FULL);
        if (!ok) break;
        const uint32_t buf = (uint32_t)(t - t_lo) & (kKsBuffers - 1);
        ok = WAIT(bar_tm_empty(buf), ((tm_par >> buf) & 1u) ^ 1u, ST_KS_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tm_par ^= 1u << buf;
        ptx::tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t d = tmem_base + buf * kTile;
          const uint32_t k_addr = s_ring + s * L::kTileBytes;
          // rows pass: lanes = queries (A = query tile); columns pass: lanes = keys (A = key tile)
          const uint32_t a_addr = PHASE == PH_ROWS ? s_q : k_addr;
          const uint32_t b_addr = PHASE == PH_ROWS ? k_addr : s_q;
          auto issue_steps = [&](auto as_tf32) {
#pragma unroll
            for (int kk = 0; kk < DPAD / 16; ++kk) {
              const uint32_t koff = (uint32_t)(kk >> 2) * L::kHalfBytes + (uint32_t)(kk & 3) * 32u;
              if constexpr (decltype(as_tf32)::value)
                ptx::umma_tf32(d, ptx::smem_desc_sw128(a_addr + koff),
                               ptx::smem_desc_sw128(b_addr + koff), p.idesc, kk > 0 ? 1u : 0u);
              else
                ptx::umma_f16(d, ptx::smem_desc_sw128(a_addr + koff),
                              ptx::smem_desc_sw128(b_addr + koff), p.idesc, kk > 0 ? 1u : 0u);
            }
          };
          if (p.tf32)
            issue_steps(std::true_type{});
          else
            issue_steps(std::false_type{});
          ptx::umma_commit(bar_tm_full(buf));
          ptx::umma_commit(bar_ring_empty(s));
        }
        __syncwarp();
      }
      if (!ok) break;
      // last item of this head on this CTA: the query tile may be replaced once these MMAs retire
      const int next_bh = (item + 1 < item_hi) ? (item + 1) / S : -1;
      if (next_bh != bh) {
        if (lane == 0) ptx::umma_commit(bar_q_empty);
        __syncwarp();
      }
    }
    if (ok && q_seq > 0) {
      // The last commit covers every MMA issued (and, in the columns pass, the barrier also
      // waits for the softmax warps): no asynchronous arrive is outstanding when the CTA retires.
      WAIT(bar_q_empty, (q_seq - 1) & 1u, ST_KS_WAIT_DRAIN);
    }
  } else {
    // -------------------------------------------------------- softmax warps
    // Warpgroup wg folds the tiles that land in accumulator buffer wg: tile t of an item goes
    // to buffer (t - t_lo) mod 4, a property of the item.
    const int wg = warp >> 2;
    const int tid_wg = (warp & 3) * 32 + lane;
    const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t taddr = tmem_base + lane_field + (uint32_t)wg * kTile;
    uint32_t my_use = 0, q_seq = 0;
    int cur_bh = -1;
    bool ok = true;
    for (int item = item_lo; ok && item < item_hi; ++item) {
      int bh, sp, t_lo, t_hi;
      keystream_item(S, p.key_tiles, item, bh, sp, t_lo, t_hi);
      if (PHASE == PH_COLS && bh != cur_bh) {
        ok = WAIT(bar_q_full, q_seq & 1u, ST_KS_WAIT_Q_FULL_SM);  // the lse values of this head
        if (!ok) break;
        ++q_seq;
      }
      cur_bh = bh;

      if constexpr (PHASE == PH_ROWS) {
        const int mine = tid_wg;  // query row
        float m_run = -INFINITY, l_run = 0.f;
        // keys j < valid_hi are attended by this query; tiles from mask_from on meet a mask edge
        const int valid_hi = p.causal ? (int)hd_min((long long)p.N, (long long)mine + p.off + 1) : p.N;
        int mask_from = p.N >> 7;
        if (p.causal) mask_from = (int)hd_min((long long)mask_from, ((long long)p.off + 1) >> 7);
        // a warp whose 32 lanes all lie beyond the last query has nothing to fold
        const bool live = (warp & 3) * 32 < p.M;
        for (int t = t_lo + wg; t < t_hi; t += kKsBuffers) {
          ok = WAIT(bar_tm_full(wg), my_use & 1u, ST_KS_WAIT_TMEM_FULL);
          if (!ok) break;
          ++my_use;
          if (!live) {
            if (lane == 0) ptx::mbar_arrive(bar_tm_empty(wg));
            __syncwarp();
            continue;
          }
          ptx::tc_fence_after_sync();
          const bool need_mask = t >= mask_from;
          const int lim_hi = valid_hi - t * kTile;
          uint32_t ra[kChunkRows];
#pragma unroll
          for (int c = 0; c < kTile / kChunkRows; ++c) {
            ptx::tmem_ld<kChunkRows>(taddr + c * kChunkRows, ra);
            ptx::tmem_ld_wait<kChunkRows>(ra);
            if (c + 1 == kTile / kChunkRows) {
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(bar_tm_empty(wg));
            }
            if (p.dump != nullptr && mine < p.M) {
              // score cache: this query's raw scores against the 64 keys of the chunk
              float4* dst = reinterpret_cast<float4*>(p.dump + ((size_t)bh * p.M + mine) * p.n_pad +
                                                      (size_t)t * kTile + c * kChunkRows);
#pragma unroll
              for (int q4 = 0; q4 < kChunkRows / 4; ++q4)
                dst[q4] = make_float4(__uint_as_float(ra[4 * q4]), __uint_as_float(ra[4 * q4 + 1]),
                                      __uint_as_float(ra[4 * q4 + 2]), __uint_as_float(ra[4 * q4 + 3]));
            }
            if (need_mask)
              rows_chunk<true, kChunkRows>(ra, p.scale2, lim_hi - kChunkRows * c, m_run, l_run);
            else
              rows_chunk<false, kChunkRows>(ra, p.scale2, kChunkRows, m_run, l_run);
          }
        }
        if (!ok) break;
        if (mine < p.M) {
          // a warpgroup without a tile in this item leaves (-inf, 0), which the combine skips
          const size_t idx = ((size_t)(sp * kKsBuffers + wg) * p.BH + bh) * p.m_pad + mine;
          p.part_m[idx] = m_run;
          p.part_l[idx] = l_run;
        }
      } else {
        const float* lse_s = reinterpret_cast<const float*>(smem + L::off_lse);
        const int n_chunks = p.fold_cols / kChunkCols;  // only the chunks that hold a query
        for (int t = t_lo + wg; t < t_hi; t += kKsBuffers) {
          ok = WAIT(bar_tm_full(wg), my_use & 1u, ST_KS_WAIT_TMEM_FULL);
          if (!ok) break;
          ++my_use;
          ptx::tc_fence_after_sync();
          const int mine = t * kTile + tid_wg;  // key column
          float acc[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[u] = (RED == RED_MAX) ? -INFINITY : 0.f;
          // queries max(mine - off, 0) <= i < M attend this key
          const int valid_lo = p.causal ? max(mine - p.off, 0) : 0;
          const bool need_mask =
              (p.M < p.fold_cols) || (p.causal && t * kTile + kTile - 1 - p.off > 0);
          uint32_t ra[kChunkCols];
          for (int c = 0; c < n_chunks; ++c) {
            ptx::tmem_ld<kChunkCols>(taddr + c * kChunkCols, ra);
            ptx::tmem_ld_wait<kChunkCols>(ra);
            if (c + 1 == n_chunks) {
              ptx::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(bar_tm_empty(wg));
            }
            if (need_mask)
              cols_chunk<RED, true, kChunkCols>(ra, lse_s + kChunkCols * c, p.scale2,
                                                valid_lo - kChunkCols * c, p.M - kChunkCols * c, acc);
            else
              cols_chunk<RED, false, kChunkCols>(ra, lse_s + kChunkCols * c, p.scale2, 0,
                                                 kChunkCols, acc);
          }
          if (mine < p.N) {
            float v;
            if (RED == RED_SUM)
              v = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            else
              v = ptx::ex2(fmaxf(fmaxf(acc[0], acc[1]), fmaxf(acc[2], acc[3])));
            if (p.mean_mode) v = v / mean_divisor(p, mine);
            store_out(p.out, p.out_dtype, (size_t)bh * p.N + mine, v);
          }
        }
        if (!ok) break;
        const int next_bh = (item + 1 < item_hi) ? (item + 1) / S : -1;
        if (next_bh != bh) {  // done with this head's lse values
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(bar_q_empty);
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
  if (warp == kKsMmaWarp) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fcr
