// Host-side planner: validates a problem and derives the launch geometry and
// workspace layout.  Pure C++ (no CUDA calls) so it can be exercised on a
// machine without a GPU.  Takes the place of the grid computation of the
// reference launcher (flash_colreduce/flash.py:286-287).
#pragma once
#include <stdint.h>

#include <algorithm>
#include <string>

#include "../../include/flash_colreduce_b200.h"

#if defined(__CUDACC__)
#define FCR_HD __host__ __device__ __forceinline__
#else
#define FCR_HD inline
#endif

namespace fcr {

constexpr int kTile = 128;            // rows per MMA tile (tensor-memory lanes)
constexpr int kSubTiles = 2;          // stationary tiles a CTA owns
constexpr int kBlockRows = kTile * kSubTiles;
constexpr int kStatusWords = 256;

// Geometry of one pass, shared by the host planner and the kernels.
struct PassGeom {
  int BH, H, M, N;
  int LS;          // stationary length: M for the rows pass, N for the columns pass
  int causal;
  int off;         // query i attends keys j <= i + off
  int n_sb;        // stationary blocks per head
  int n_split;     // splits of the streamed range
  int n_items;     // BH * n_sb * n_split
  int sb_reverse;  // heaviest blocks first
  int head_group;  // heads whose items are interleaved (their Q and K share the L2 cache)
};

// One work item: a head, a block of two stationary 128-row tiles, one split of
// the streamed range.  Tiles [t_lo[a], t_hi[a]) are multiplied against
// stationary sub-tile a; the item streams tiles [c_lo, c_hi).
struct Item {
  int bh, sp;
  int par;  // parity of the item's index: which accumulator buffer its first tile uses
  int r0[kSubTiles];
  int t_lo[kSubTiles], t_hi[kSubTiles];
  int c_lo, c_hi;
};

// Key streaming: work item `item` of either pass is chunk item % S of head item / S and covers
// key tiles [key_tiles * sp / S, key_tiles * (sp + 1) / S) of that head.
FCR_HD void keystream_item(int S, int key_tiles, int item, int& bh, int& sp, int& t_lo, int& t_hi) {
  bh = item / S;
  sp = item - bh * S;
  t_lo = (int)(((long long)key_tiles * sp) / S);
  t_hi = (int)(((long long)key_tiles * (sp + 1)) / S);
}

template <typename T>
FCR_HD T hd_min(T a, T b) { return a < b ? a : b; }
template <typename T>
FCR_HD T hd_max(T a, T b) { return a > b ? a : b; }

// Maps a linear work-item index to its head, stationary block and split, and
// derives the streamed tile range of each stationary sub-tile.  The rows pass
// keeps Q tiles stationary and streams the K tiles a tile's rows may attend;
// the columns pass keeps K tiles stationary and streams the Q tiles that may
// attend them.  Fully masked tiles are in no range (the reference skips them
// per 64-row program, flash_colreduce/flash.py:201-207).
template <bool COLS>
FCR_HD Item decode_item(const PassGeom& p, int item) {
  // Item order: groups of `head_group` heads; inside a group the stationary
  // blocks run heaviest first and the heads of the group are interleaved, so
  // that concurrently running CTAs work on few heads (L2 reuse of the streamed
  // operand) while the work handed out last is the lightest (short tail).
  Item g;
  const int sp = item % p.n_split;
  const int rest = item / p.n_split;
  const int per_group = p.head_group * p.n_sb;
  const int grp = rest / per_group;
  const int in_grp = rest - grp * per_group;
  const int heads_here = hd_min(p.head_group, p.BH - grp * p.head_group);
  const int o = in_grp / heads_here;
  g.bh = grp * p.head_group + (in_grp - o * heads_here);
  g.sp = sp;
  g.par = item & 1;
  const int sb = p.sb_reverse ? (p.n_sb - 1 - o) : o;
  int lo = 0x7fffffff, hi = 0;
  int tb[kSubTiles], te[kSubTiles];
#if defined(__CUDACC__)
#pragma unroll
#endif
  for (int a = 0; a < kSubTiles; ++a) {
    const int r0 = (sb * kSubTiles + a) * kTile;
    g.r0[a] = r0;
    tb[a] = 0;
    te[a] = 0;
    if (r0 < p.LS) {
      if (COLS) {
        te[a] = (p.M + kTile - 1) / kTile;
        if (p.causal) {
          const int imin = hd_max(r0 - p.off, 0);  // first query that sees key r0
          tb[a] = hd_min(imin / kTile, te[a]);
        }
      } else {
        long long jmax = (long long)p.N - 1;
        if (p.causal) {
          const long long last_row = (long long)hd_min(r0 + kTile, p.M) - 1;
          jmax = hd_min(jmax, last_row + p.off);
        }
        te[a] = (int)(jmax / kTile) + 1;
      }
      lo = hd_min(lo, tb[a]);
      hi = hd_max(hi, te[a]);
    }
  }
  if (lo > hi) lo = hi;
  const long long len = hi - lo;
  g.c_lo = lo + (int)((len * sp) / p.n_split);
  g.c_hi = lo + (int)((len * (sp + 1)) / p.n_split);
#if defined(__CUDACC__)
#pragma unroll
#endif
  for (int a = 0; a < kSubTiles; ++a) {
    g.t_lo[a] = hd_max(tb[a], g.c_lo);
    g.t_hi[a] = hd_max(hd_min(te[a], g.c_hi), g.t_lo[a]);
    if (g.r0[a] >= p.LS) {
      g.t_lo[a] = g.c_lo;
      g.t_hi[a] = g.c_lo;
    }
  }
  return g;
}

inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t align_up64(int64_t a, int64_t b) { return ceil_div64(a, b) * b; }

// Number of keys query row i attends (flash_colreduce/flash.py:22-27, naive.py:20-24).
inline int64_t valid_keys(int64_t i, int64_t N, bool causal, int64_t off) {
  if (!causal) return N;
  return std::min<int64_t>(i + off + 1, N);
}

inline int choose_splits(int64_t base_items, int64_t max_len_tiles, int num_sms) {
  // Splitting the streamed range of an item S ways shortens the critical path of a small
  // problem (more CTAs work in parallel) but costs a combine kernel and per-item set-up.
  // Cost model in units of one streamed tile step: every item pays 2 steps of set-up,
  // the combine launch about 3; items run in waves of num_sms.  Large problems (at least
  // one full wave without splitting) never split.
  int best = 1;
  int64_t best_cost = -1;
  for (int s = 1; s <= 64 && s <= max_len_tiles; s *= 2) {
    const int64_t waves = ceil_div64(base_items * s, num_sms);
    const int64_t cost = waves * (ceil_div64(max_len_tiles, s) + 2) + (s > 1 ? 3 : 0);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = s;
    }
    if (base_items * s >= num_sms) break;  // the grid is full: more splits only add overhead
  }
  return best;
}

inline int plan_problem(const fcr_problem& p, int num_sms, fcr_plan& pl, std::string& err) {
  pl = fcr_plan{};
  if (p.B <= 0 || p.H <= 0 || p.M <= 0 || p.N <= 0 || p.D <= 0) {
    err = "B, H, M, N and D must all be positive";
    return FCR_ERR_BAD_ARG;
  }
  if (p.reduction != FCR_SUM && p.reduction != FCR_MEAN && p.reduction != FCR_MAX) {
    err = "invalid reduction code " + std::to_string(p.reduction);
    return FCR_ERR_BAD_ARG;
  }
  if (p.in_dtype != FCR_F16 && p.in_dtype != FCR_BF16 && p.in_dtype != FCR_F32) {
    err = "q and k must be fp16, bf16 or fp32 (dtype code " + std::to_string(p.in_dtype) + ")";
    return FCR_ERR_UNSUPPORTED;
  }
  // An operand row may span at most 512 bytes (four 128-byte swizzled slabs).
  const int elem_bytes = p.in_dtype == FCR_F32 ? 4 : 2;
  const int align_elems = 16 / elem_bytes;  // strides must be multiples of 16 bytes
  if (p.D * elem_bytes > 512) {
    err = "head dimension " + std::to_string(p.D) + " exceeds " + std::to_string(512 / elem_bytes) +
          " (operand rows of at most 512 bytes)";
    return FCR_ERR_UNSUPPORTED;
  }
  if (p.M > (1 << 30) || p.N > (1 << 30)) {
    err = "M and N are limited to 2^30";
    return FCR_ERR_UNSUPPORTED;
  }
  for (int t = 0; t < 2; ++t) {
    const int64_t* s = t ? p.k_strides : p.q_strides;
    const char* name = t ? "k" : "q";
    if (s[3] != 1) {
      err = std::string(name) + ": innermost stride must be 1";
      return FCR_ERR_UNSUPPORTED;
    }
    const int32_t dims[3] = {p.B, p.H, t ? p.N : p.M};
    for (int a = 0; a < 3; ++a) {
      if (dims[a] > 1 && (s[a] <= 0 || s[a] % align_elems != 0)) {
        err = std::string(name) + ": stride " + std::to_string(a) + " = " + std::to_string(s[a]) +
              " is not a positive multiple of " + std::to_string(align_elems) + " elements (16 bytes)";
        return FCR_ERR_UNSUPPORTED;
      }
    }
  }
  if (num_sms <= 0) {
    err = "num_sms must be positive";
    return FCR_ERR_BAD_ARG;
  }
  const bool causal = p.is_causal != 0;
  const int64_t off = !causal ? 0
                      : (p.causal_offset >= 0 ? p.causal_offset
                                              : std::max<int64_t>((int64_t)p.N - p.M, 0));
  if (off > (1LL << 30)) {
    err = "causal_offset too large";
    return FCR_ERR_BAD_ARG;
  }
  const int64_t BH = (int64_t)p.B * p.H;

  // row width the kernels run at, in 2-byte units: 128, 256 or 512 bytes
  pl.d_pad = p.D * elem_bytes <= 128 ? 64 : (p.D * elem_bytes <= 256 ? 128 : 256);
  pl.rows_per_block = kBlockRows;
  pl.m_pad = (int32_t)align_up64(p.M, kTile);
  pl.n_pad = (int32_t)align_up64(p.N, kTile);
  pl.causal_offset = off;
  pl.row_blocks = (int32_t)ceil_div64(p.M, kBlockRows);
  pl.col_blocks = (int32_t)ceil_div64(p.N, kBlockRows);

  // Longest streamed range of any block, in tiles.
  const int64_t keys_seen = causal ? std::min<int64_t>(p.N, (int64_t)p.M + off) : p.N;
  const int64_t row_len = ceil_div64(keys_seen, kTile);
  const int64_t col_len = ceil_div64(p.M, kTile);
  pl.row_splits = choose_splits(BH * pl.row_blocks, row_len, num_sms);
  pl.col_splits = choose_splits(BH * pl.col_blocks, col_len, num_sms);
  const int64_t row_items = BH * pl.row_blocks * pl.row_splits;
  const int64_t col_items = BH * pl.col_blocks * pl.col_splits;
  if (row_items > (1LL << 30) || col_items > (1LL << 30)) {
    err = "problem has too many work items";
    return FCR_ERR_UNSUPPORTED;
  }
  pl.row_items = (int32_t)row_items;
  pl.col_items = (int32_t)col_items;
  // With the causal mask the items of a head shrink towards its end: interleave the
  // heads whose Q and K (fp16) total at most 128 MiB (32 heads at most; measured flat from 16 to 32),
  // so that the tail of the grid is made of the lightest items of many heads.  Without
  // the mask all items weigh the same and one head at a time keeps the CTAs in step.
  const int64_t head_bytes = ((int64_t)p.M + p.N) * pl.d_pad * 2;
  pl.head_group = !causal ? 1
                          : (int32_t)std::max<int64_t>(
                                1, std::min<int64_t>(std::min<int64_t>(BH, 32), (128LL << 20) / head_bytes));
  // Items that stream at most 8 tiles get the double-buffered stationary stage.
  pl.short_items = (ceil_div64(row_len, pl.row_splits) <= 8 ? 1 : 0) |
                   (ceil_div64(col_len, pl.col_splits) <= 8 ? 2 : 0);
  pl.row_ctas = (int32_t)std::min<int64_t>(row_items, num_sms);
  pl.col_ctas = (int32_t)std::min<int64_t>(col_items, num_sms);

  // Decode shapes: every query of a head fits one tile and the keys are long.  Both passes then
  // stream the key tiles (see keystream_item); CTA c runs items [c*I/G, (c+1)*I/G), so S is
  // chosen to minimise the longest CTA: items per CTA times (tiles per item + one tile of
  // per-item overhead).
  pl.key_stream = 0;
  pl.key_chunks = 0;
  const int64_t key_tiles = pl.n_pad / kTile;
  if (pl.m_pad == kTile && key_tiles >= 8) {
    int best_s = 1;
    int64_t best_cost = -1;
    for (int64_t s = 1; s <= std::min<int64_t>(key_tiles, 256); ++s) {
      const int64_t per_cta = ceil_div64(BH * s, num_sms);
      const int64_t cost = per_cta * (ceil_div64(key_tiles, s) + 1);
      if (best_cost < 0 || cost < best_cost) {
        best_cost = cost;
        best_s = (int)s;
      }
    }
    if (BH * best_s > (1LL << 30)) {
      err = "problem has too many work items";
      return FCR_ERR_UNSUPPORTED;
    }
    pl.key_stream = 1;
    pl.key_chunks = best_s;
    pl.row_splits = 4 * best_s;  // one partial state per chunk and softmax warpgroup
    pl.col_splits = 1;
    pl.row_items = pl.col_items = (int32_t)(BH * best_s);
    pl.row_ctas = pl.col_ctas = (int32_t)std::min<int64_t>(pl.row_items, num_sms);
    pl.head_group = 1;
    pl.short_items = 0;
  }

  // Small problems (at most two work items per CTA) deal their items round-robin: no work
  // counter, so nothing in the workspace needs clearing before the kernels.  The key-streaming
  // kernels never use the counter.
  pl.static_schedule = (pl.key_stream || (pl.row_items <= 2 * pl.row_ctas && pl.col_items <= 2 * pl.col_ctas)) ? 1 : 0;

  int64_t scores = 0;
  if (!causal) {
    scores = (int64_t)p.M * p.N;
  } else {
    // rows i < N - off see i + off + 1 keys, the rest see N
    const int64_t ramp = std::max<int64_t>(0, std::min<int64_t>(p.M, (int64_t)p.N - off));
    scores = ramp * (off + 1) + ramp * (ramp - 1) / 2 + ((int64_t)p.M - ramp) * p.N;
  }
  pl.valid_scores = scores * BH;

  int64_t o = 0;
  pl.off_status = o;
  o += align_up64(kStatusWords * 4, 256);
  pl.off_neg_lse = o;
  o += align_up64(BH * pl.m_pad * 4, 256);
  if (pl.row_splits > 1) {
    pl.off_part_m = o;
    o += align_up64((int64_t)pl.row_splits * BH * pl.m_pad * 4, 256);
    pl.off_part_l = o;
    o += align_up64((int64_t)pl.row_splits * BH * pl.m_pad * 4, 256);
  }
  if (pl.col_splits > 1) {
    pl.off_part_out = o;
    o += align_up64((int64_t)pl.col_splits * BH * pl.n_pad * 4, 256);
  }
  // Decode with a handful of queries: 4*M bytes of scores per key are far fewer than the key's
  // own bytes, so the rows pass keeps them and the second sweep over K is not needed.
  const int64_t score_bytes = BH * p.M * (int64_t)pl.n_pad * 4;
  if (pl.key_stream && p.M <= 16 && score_bytes <= (1LL << 31)) {
    pl.score_cache = 1;
    pl.off_scores = o;
    o += align_up64(score_bytes, 256);
  }
  pl.workspace_bytes = o;
  return FCR_OK;
}

// Geometry of the rows pass (cols == false) or the columns pass of a plan.
inline PassGeom pass_geometry(const fcr_problem& p, const fcr_plan& pl, bool cols) {
  PassGeom g{};
  g.BH = p.B * p.H;
  g.H = p.H;
  g.M = p.M;
  g.N = p.N;
  g.causal = p.is_causal ? 1 : 0;
  g.off = (int)pl.causal_offset;
  g.LS = cols ? p.N : p.M;
  g.n_sb = cols ? pl.col_blocks : pl.row_blocks;
  g.n_split = cols ? pl.col_splits : pl.row_splits;
  g.n_items = cols ? pl.col_items : pl.row_items;
  g.sb_reverse = (!cols && g.causal) ? 1 : 0;  // rows pass: late blocks see the most keys
  g.head_group = pl.head_group;
  return g;
}

}  // namespace fcr
