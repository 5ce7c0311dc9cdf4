// Per-thread folds of the two passes: a softmax thread owns one accumulator
// row (one tensor-memory lane) and folds W of its columns at a time.
#pragma once
#include <math.h>
#include <stdint.h>

#include "ptx_sm100.cuh"

namespace fcr {

enum { RED_SUM = 0, RED_MAX = 1 };

#ifndef FCR_POLY
#define FCR_POLY 2
#endif
// Pairs of exponentials, out of every 8 pairs (16 elements), that are evaluated by the
// polynomial on the FMA pipe instead of MUFU: 2 = a quarter of all exponentials.
constexpr int kPolyOf8 = FCR_POLY;
#ifndef FCR_POLY_ROWS
#define FCR_POLY_ROWS FCR_POLY
#endif
#ifndef FCR_POLY_COLS
#define FCR_POLY_COLS FCR_POLY
#endif
constexpr int kPolyRows = FCR_POLY_ROWS;  // the share in the rows pass
constexpr int kPolyCols = FCR_POLY_COLS;  // the share in the columns pass (sum / mean)
// Spreads POLY chosen pairs evenly over each group of 8 pairs.
__host__ __device__ constexpr bool poly_pair(int e, int poly) { return ((((e & 15) >> 1) * poly) & 7) < poly; }

// ---------------------------------------------------------------- rows pass
// One 32-column chunk of a query row: online max / sum in the base-2 domain
// (flash_colreduce/flash.py:71-78).  `nvalid` = number of leading columns of
// the chunk this row may attend (only read when MASKED).
template <bool MASKED, int W, int POLY = kPolyRows>
__device__ __forceinline__ void rows_chunk(const uint32_t* r, float scale2, int nvalid,
                                           float& m_run, float& l_run) {
  float x[W];
#pragma unroll
  for (int e = 0; e < W; ++e) {
    x[e] = __uint_as_float(r[e]);
    if (MASKED && e >= nvalid) x[e] = -INFINITY;
  }
  float mx0 = ptx::max3(x[0], x[1], x[2]), mx1 = ptx::max3(x[3], x[4], x[5]);
  mx0 = fmaxf(mx0, x[6]);
  mx1 = fmaxf(mx1, x[7]);
#pragma unroll
  for (int e = 8; e < W; e += 4) {
    mx0 = ptx::max3(mx0, x[e], x[e + 1]);
    mx1 = ptx::max3(mx1, x[e + 2], x[e + 3]);
  }
  const float m_new = fmaxf(m_run, fmaxf(mx0, mx1) * scale2);
  const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;  // row sees nothing yet
  const float alpha = ptx::ex2(m_run - m_safe);
  const float nm = -m_safe;
  float2 s01 = make_float2(0.f, 0.f), s23 = make_float2(0.f, 0.f);
#pragma unroll
  for (int e = 0; e < W; e += 4) {
    float2 a01 = __ffma2_rn(make_float2(x[e], x[e + 1]), make_float2(scale2, scale2),
                            make_float2(nm, nm));
    float2 a23 = __ffma2_rn(make_float2(x[e + 2], x[e + 3]), make_float2(scale2, scale2),
                            make_float2(nm, nm));
    // kPolyOf8 of every 8 exponentials are evaluated on the FMA pipe (never in masked tiles)
    if (!MASKED && poly_pair(e, POLY)) {
      a01 = ptx::ex2_poly2(a01);
    } else {
      a01.x = ptx::ex2(a01.x);
      a01.y = ptx::ex2(a01.y);
    }
    if (!MASKED && poly_pair(e + 2, POLY)) {
      a23 = ptx::ex2_poly2(a23);
    } else {
      a23.x = ptx::ex2(a23.x);
      a23.y = ptx::ex2(a23.y);
    }
    s01 = __fadd2_rn(s01, a01);
    s23 = __fadd2_rn(s23, a23);
  }
  l_run = fmaf(l_run, alpha, (s01.x + s01.y) + (s23.x + s23.y));
  m_run = m_new;
}

// ------------------------------------------------------------- columns pass
// One 32-query chunk of a key column: P = exp2(s*scale2 - lse_i) folded into
// the column's accumulators (flash_colreduce/flash.py:120-124).  Queries
// e in [e_lo, e_hi) of the chunk are valid (only read when MASKED).  For max
// the fold is done on the exponent, exp2 being monotonic.
template <int RED, bool MASKED, int W, int POLY = kPolyCols>
__device__ __forceinline__ void cols_chunk(const uint32_t* r, const float* neg_lse,
                                           float scale2, int e_lo, int e_hi, float (&acc)[4]) {
#pragma unroll
  for (int q = 0; q < W / 4; ++q) {
    const float4 nl = reinterpret_cast<const float4*>(neg_lse)[q];
    const int e = q * 4;
    float2 t01 = __ffma2_rn(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])),
                            make_float2(scale2, scale2), make_float2(nl.x, nl.y));
    float2 t23 = __ffma2_rn(make_float2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3])),
                            make_float2(scale2, scale2), make_float2(nl.z, nl.w));
    if (RED == RED_SUM) {
      // kPolyOf8 of every 8 exponentials are evaluated on the FMA pipe (never in masked tiles)
      if (!MASKED && poly_pair(e, POLY)) {
        t01 = ptx::ex2_poly2(t01);
      } else {
        t01.x = ptx::ex2(t01.x);
        t01.y = ptx::ex2(t01.y);
      }
      if (!MASKED && poly_pair(e + 2, POLY)) {
        t23 = ptx::ex2_poly2(t23);
      } else {
        t23.x = ptx::ex2(t23.x);
        t23.y = ptx::ex2(t23.y);
      }
      if (MASKED) {
        t01.x = (e >= e_lo && e < e_hi) ? t01.x : 0.f;
        t01.y = (e + 1 >= e_lo && e + 1 < e_hi) ? t01.y : 0.f;
        t23.x = (e + 2 >= e_lo && e + 2 < e_hi) ? t23.x : 0.f;
        t23.y = (e + 3 >= e_lo && e + 3 < e_hi) ? t23.y : 0.f;
      }
      // packed adds: acc[0..1] and acc[2..3] are two register pairs
      const float2 a01 = __fadd2_rn(make_float2(acc[0], acc[1]), t01);
      const float2 a23 = __fadd2_rn(make_float2(acc[2], acc[3]), t23);
      acc[0] = a01.x;
      acc[1] = a01.y;
      acc[2] = a23.x;
      acc[3] = a23.y;
    } else {
      if (MASKED) {
        t01.x = (e >= e_lo && e < e_hi) ? t01.x : -INFINITY;
        t01.y = (e + 1 >= e_lo && e + 1 < e_hi) ? t01.y : -INFINITY;
        t23.x = (e + 2 >= e_lo && e + 2 < e_hi) ? t23.x : -INFINITY;
        t23.y = (e + 3 >= e_lo && e + 3 < e_hi) ? t23.y : -INFINITY;
      }
      acc[0] = ptx::max3(acc[0], t01.x, t01.y);
      acc[1] = ptx::max3(acc[1], t23.x, t23.y);
    }
  }
}

}  // namespace fcr
