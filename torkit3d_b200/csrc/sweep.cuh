// Filter-then-verify sweep over a key cloud for fp32 queries.
//
// All three O(N*M) operators (nearest neighbour, k nearest neighbours, ball query) must decide
// with the exactly rounded squared distance
//     d = ((dx*dx + dy*dy) + dz*dz),  dx = key.x - query.x,  no fused multiply-add,
// which costs 8 FP32 instructions per pair.  The sweep evaluates a cheaper LOWER-BOUND test with
// three fused multiply-adds and one compare per pair and only recomputes d for the pairs that
// pass it.  The decision is always taken on d, so results are bit-identical to the plain loop; the
// filter only has to be conservative.
//
// Per key point the tile holds (x, y, z, w) with  w = fl(|r|^2 * (1 - 12u)),  u = 2^-24.
// Per query the thread holds m = -2 q (exact) and a threshold t.  For a pair
//     a = fma(m.x, r.x, fma(m.y, r.y, fma(m.z, r.z, w)))
// and with A = |r|^2 - 2 q.r (real arithmetic), P = |r|^2 + 2 sum|q_c r_c| <= 2|r|^2 + |q|^2:
//     w  <= |r|^2 (1+3u)(1-12u)(1+u) <= |r|^2 (1 - 7.9u)      (|r|^2 summed with three roundings)
//     a  <= (w - 2 q.r) + 3u P (1 + O(u))  <=  A + 3.01u |q|^2 (the |r|^2 terms cancel: -7.9u + 6u < 0)
// The exactly rounded d satisfies d >= D (1 - 5.01u), D = A + |q|^2.  Hence for a bound `lim`
//     d < lim   ==>   a < lim (1 + 5.1u) - |q|^2 (1 - 3.01u)
// threshold(lim, qq) below returns a float that is >= that right-hand side including the rounding
// of its own three operations and of qq = fl(|q|^2) (16u on both terms, plus an absolute slack for
// gradual underflow), so  "a < t" can never reject a pair with d < lim.  The test is written
// !(a >= t) so that a NaN or inf produced by enormous coordinates falls into the verify path.
#pragma once

#include "tk3d_common.cuh"

namespace tk3d {

__device__ __forceinline__ float sweep_key_w(float x, float y, float z) {
  const float rr = fmaf(z, z, fmaf(y, y, x * x));
  return rr * (1.0f - 12.0f * 5.9604645e-8f);
}

__device__ __forceinline__ float sweep_threshold(float lim, float qq) {
  const float up = 1.0f + 16.0f * 5.9604645e-8f;   // exactly representable
  const float dn = 1.0f - 16.0f * 5.9604645e-8f;   // exactly representable
  return __fadd_rn(__fsub_rn(__fmul_rn(lim, up), __fmul_rn(qq, dn)), 1e-37f);
}

__device__ __forceinline__ float sweep_qq(float x, float y, float z) { return fmaf(z, z, fmaf(y, y, x * x)); }

// Stage `count` key points starting at `src` (array of xyz triples) into `dst` as (x,y,z,w).
// Slots beyond `count` up to `padded` get a point that can never pass a filter (w = +inf gives
// a = +inf or NaN; callers bound their loops by `count`, the padding only keeps LDS in range).
template <int THREADS>
__device__ __forceinline__ void sweep_stage_tile(float4 *dst, const float *__restrict__ src, int count, int tid) {
  for (int u = tid; u < count; u += THREADS) {
    const float x = src[u * 3 + 0], y = src[u * 3 + 1], z = src[u * 3 + 2];
    dst[u] = make_float4(x, y, z, sweep_key_w(x, y, z));
  }
}

}  // namespace tk3d
