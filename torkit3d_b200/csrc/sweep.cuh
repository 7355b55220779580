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

// "Does any of the eight filter values fall below its threshold?"  Written in PTX so that the
// eight compares chain through ONE predicate (setp.ltu.or) and a single branch follows; left to
// the compiler, each compare becomes its own branch.  ltu = "less than or unordered", i.e.
// !(a >= t): a NaN on either side counts as a pass.
__device__ __forceinline__ bool sweep_any8(float a0, float a1, float a2, float a3, float a4, float a5, float a6,
                                           float a7, float t0, float t1, float t2, float t3, float t4, float t5,
                                           float t6, float t7) {
  unsigned flag;
  asm("{\n\t"
      ".reg .pred p;\n\t"
      "setp.ltu.f32 p, %1, %9;\n\t"
      "setp.ltu.or.f32 p, %2, %10, p;\n\t"
      "setp.ltu.or.f32 p, %3, %11, p;\n\t"
      "setp.ltu.or.f32 p, %4, %12, p;\n\t"
      "setp.ltu.or.f32 p, %5, %13, p;\n\t"
      "setp.ltu.or.f32 p, %6, %14, p;\n\t"
      "setp.ltu.or.f32 p, %7, %15, p;\n\t"
      "setp.ltu.or.f32 p, %8, %16, p;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(flag)
      : "f"(a0), "f"(a1), "f"(a2), "f"(a3), "f"(a4), "f"(a5), "f"(a6), "f"(a7), "f"(t0), "f"(t1), "f"(t2), "f"(t3),
        "f"(t4), "f"(t5), "f"(t6), "f"(t7));
  return flag != 0;
}

// Filter values of one key against Q queries.
__device__ __forceinline__ float sweep_lower(float mx, float my, float mz, const float4 &r) {
  return fmaf(mx, r.x, fmaf(my, r.y, fmaf(mz, r.z, r.w)));
}

// Eight filter values for a group of 8/Q consecutive keys x Q queries, and the combined test.
// a[u*Q + s] belongs to key u of the group and query s.
template <int Q>
__device__ __forceinline__ bool sweep_group(const float4 *__restrict__ keys, const float (&mx)[Q],
                                            const float (&my)[Q], const float (&mz)[Q], const float (&thr)[Q],
                                            float (&a)[8]) {
  constexpr int U = 8 / Q;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const float4 r = keys[u];
#pragma unroll
    for (int s = 0; s < Q; ++s) a[u * Q + s] = sweep_lower(mx[s], my[s], mz[s], r);
  }
  return sweep_any8(a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], thr[0 % Q], thr[1 % Q], thr[2 % Q], thr[3 % Q],
                    thr[4 % Q], thr[5 % Q], thr[6 % Q], thr[7 % Q]);
}

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
