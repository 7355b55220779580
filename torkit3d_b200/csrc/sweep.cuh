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
//     a = fma(m.x, r.x, fma(m.y, r.y, fma(m.z, r.z, w)))      (scalar or packed FMAs alike)
// and with A = |r|^2 - 2 q.r (real arithmetic), P = |r|^2 + 2 sum|q_c r_c| <= 2|r|^2 + |q|^2:
//     w  <= |r|^2 (1+3u)(1-12u)(1+u) <= |r|^2 (1 - 7.9u)      (|r|^2 summed with three roundings)
//     a  <= (w - 2 q.r) + 3u P (1 + O(u))  <=  A + 3.01u |q|^2 (the |r|^2 terms cancel: -7.9u + 6u < 0)
// The exactly rounded d satisfies d >= D (1 - 5.01u), D = A + |q|^2.  Hence for a bound `lim`
//     d < lim   ==>   a < lim (1 + 5.1u) - |q|^2 (1 - 3.01u)
// threshold(lim, qq) below returns a float that is >= that right-hand side including the rounding
// of its own three operations and of qq = fl(|q|^2) (16u on both terms, plus an absolute slack for
// gradual underflow), so  "a < t" can never reject a pair with d < lim.
// Non-finite values.  Coordinates beyond about 1e19 overflow |r|^2, |q|^2 or q.r although the
// distance of two such points can be finite.  The tests are therefore written "a < t or unordered"
// (!(a >= t)): a NaN filter value (inf - inf) reaches the verify path, -inf passes, and +inf only
// arises where the exact distance is infinite too.  |q|^2 and the key term w are clamped to the
// largest finite float (sweep_qq, sweep_key_w), so that a threshold is never NaN or -inf for a real
// query and a real key never carries the +inf that marks padding.  Key tiles are padded with
// (0, 0, 0, w = +inf): a padding key's filter value is +inf, which no threshold admits, so the
// verify paths need no bounds test.  A threshold of +inf means "accept every real key", -inf
// "accept nothing".
#pragma once

#include "tk3d_common.cuh"

namespace tk3d {

__device__ __forceinline__ float sweep_key_w(float x, float y, float z) {
  const float rr = fmaf(z, z, fmaf(y, y, x * x));
  // Clamped to the largest finite float: an overflowed |r|^2 must not turn the filter value into
  // +inf ("never passes") for a key whose distance is finite; too small a w only passes more keys.
  return fminf(rr * (1.0f - 12.0f * 5.9604645e-8f), 3.402823466e38f);
}

__device__ __forceinline__ float sweep_threshold(float lim, float qq) {
  const float up = 1.0f + 16.0f * 5.9604645e-8f;   // exactly representable
  const float dn = 1.0f - 16.0f * 5.9604645e-8f;   // exactly representable
  return __fadd_rn(__fsub_rn(__fmul_rn(lim, up), __fmul_rn(qq, dn)), 1e-37f);
}

__device__ __forceinline__ float sweep_qq(float x, float y, float z) {
  return fminf(fmaf(z, z, fmaf(y, y, x * x)), 3.402823466e38f);  // NaN and +inf become FLT_MAX
}

// "Does any of the eight filter values fall below its threshold?"  Written in PTX so that the
// eight compares chain through two predicates (setp.ltu.or) that are OR-ed once, and a single
// branch follows; left to the compiler, each compare becomes its own branch.  ltu = "less than or unordered", i.e.
// !(a >= t): a NaN on either side counts as a pass.
__device__ __forceinline__ bool sweep_any8(float a0, float a1, float a2, float a3, float a4, float a5, float a6,
                                           float a7, float t0, float t1, float t2, float t3, float t4, float t5,
                                           float t6, float t7) {
  unsigned flag;
  asm("{\n\t"
      ".reg .pred p;\n\t"
      ".reg .pred q;\n\t"
      "setp.ltu.f32 p, %1, %9;\n\t"
      "setp.ltu.f32 q, %2, %10;\n\t"
      "setp.ltu.or.f32 p, %3, %11, p;\n\t"
      "setp.ltu.or.f32 q, %4, %12, q;\n\t"
      "setp.ltu.or.f32 p, %5, %13, p;\n\t"
      "setp.ltu.or.f32 q, %6, %14, q;\n\t"
      "setp.ltu.or.f32 p, %7, %15, p;\n\t"
      "setp.ltu.or.f32 q, %8, %16, q;\n\t"
      "or.pred p, p, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(flag)
      : "f"(a0), "f"(a1), "f"(a2), "f"(a3), "f"(a4), "f"(a5), "f"(a6), "f"(a7), "f"(t0), "f"(t1), "f"(t2), "f"(t3),
        "f"(t4), "f"(t5), "f"(t6), "f"(t7));
  return flag != 0;
}

// The same question asked through minima: three-input minima (one instruction each on sm_100)
// feed one compare per query, which takes most of the compares off the half-rate pipe.  The minima
// propagate NaN and the compare is "less than or unordered", so a NaN filter value (inf - inf, when
// |r|^2 or q.r overflow although the distance itself is finite) still reaches the verify path.
__device__ __forceinline__ float sweep_min3(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// v0..v3 against t0, v4..v7 against t1.
__device__ __forceinline__ bool sweep_any8_min(float v0, float v1, float v2, float v3, float v4, float v5, float v6,
                                               float v7, float t0, float t1) {
  unsigned flag;
  asm("{\n\t"
      ".reg .pred p;\n\t"
      ".reg .f32 m0;\n\t"
      ".reg .f32 m1;\n\t"
      "min.NaN.f32 m0, %1, %2, %3;\n\t"
      "min.NaN.f32 m1, %5, %6, %7;\n\t"
      "min.NaN.f32 m0, m0, %4;\n\t"
      "min.NaN.f32 m1, m1, %8;\n\t"
      "setp.ltu.f32 p, m0, %9;\n\t"
      "setp.ltu.or.f32 p, m1, %10, p;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(flag)
      : "f"(v0), "f"(v1), "f"(v2), "f"(v3), "f"(v4), "f"(v5), "f"(v6), "f"(v7), "f"(t0), "f"(t1));
  return flag != 0;
}

// As sweep_any8_min, and the two minima themselves (m0 over v0..v3, m1 over v4..v7) for callers
// that gate their verify path per query.
__device__ __forceinline__ bool sweep_any8_min2(float v0, float v1, float v2, float v3, float v4, float v5, float v6,
                                                float v7, float t0, float t1, float &m0, float &m1) {
  unsigned flag;
  asm("{\n\t"
      ".reg .pred p;\n\t"
      "min.NaN.f32 %1, %3, %4, %5;\n\t"
      "min.NaN.f32 %2, %7, %8, %9;\n\t"
      "min.NaN.f32 %1, %1, %6;\n\t"
      "min.NaN.f32 %2, %2, %10;\n\t"
      "setp.ltu.f32 p, %1, %11;\n\t"
      "setp.ltu.or.f32 p, %2, %12, p;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(flag), "=&f"(m0), "=&f"(m1)
      : "f"(v0), "f"(v1), "f"(v2), "f"(v3), "f"(v4), "f"(v5), "f"(v6), "f"(v7), "f"(t0), "f"(t1));
  return flag != 0;
}

// Filter values of one key against Q queries.
__device__ __forceinline__ float sweep_lower(float mx, float my, float mz, const float4 &r) {
  return fmaf(mx, r.x, fmaf(my, r.y, fmaf(mz, r.z, r.w)));
}

// ---- key tiles in "pair" layout, for the packed FP32 instructions of sm_100 ------------------------
// Two consecutive keys (2p, 2p+1) occupy two float4 slots:
//     tile[2p]   = (x0, x1, y0, y1)      tile[2p+1] = (z0, z1, w0, w1)
// so that one fma.rn.f32x2 (FFMA2) evaluates the filter of one query against BOTH keys: the
// query's multipliers are held duplicated, (m, m), in 64-bit register pairs.  A packed FMA takes
// one issue slot and three 64-bit register reads for two FMAs, which relieves the issue and
// register-file limits that cap the scalar loop well below the FMA rate.
__device__ __forceinline__ void sweep_store_key(float4 *tile, int u, float x, float y, float z, float w) {
  float *f = reinterpret_cast<float *>(tile) + (u >> 1) * 8 + (u & 1);
  f[0] = x;
  f[2] = y;
  f[4] = z;
  f[6] = w;
}

__device__ __forceinline__ float4 sweep_load_key(const float4 *tile, int u) {
  const float *f = reinterpret_cast<const float *>(tile) + (u >> 1) * 8 + (u & 1);
  return make_float4(f[0], f[2], f[4], f[6]);
}

// Filter values of a group of 4/Q key pairs (8/Q keys) x Q queries: a[p*Q + s] = (value for key
// 2p, value for key 2p+1) of query s; returns "any of the eight passes".  `pairs` points at the
// first float4 slot of the group (slot index = key index, which must be even).
template <int Q, bool MINV = false>
__device__ __forceinline__ bool sweep_group2(const float4 *__restrict__ pairs, const float2 (&mx)[Q],
                                             const float2 (&my)[Q], const float2 (&mz)[Q], const float (&thr)[Q],
                                             float2 (&a)[4]) {
  static_assert(Q == 1 || Q == 2 || Q == 4, "eight (key, query) pairs per group");
  constexpr int P = 4 / Q;
#pragma unroll
  for (int p = 0; p < P; ++p) {
    const float4 A = pairs[2 * p], Bv = pairs[2 * p + 1];
    const float2 kx = make_float2(A.x, A.y), ky = make_float2(A.z, A.w);
    const float2 kz = make_float2(Bv.x, Bv.y), kw = make_float2(Bv.z, Bv.w);
#pragma unroll
    for (int s = 0; s < Q; ++s) a[p * Q + s] = __ffma2_rn(mx[s], kx, __ffma2_rn(my[s], ky, __ffma2_rn(mz[s], kz, kw)));
  }
  if constexpr (MINV && Q == 2)  // a[0], a[2] belong to query 0; a[1], a[3] to query 1
    return sweep_any8_min(a[0].x, a[0].y, a[2].x, a[2].y, a[1].x, a[1].y, a[3].x, a[3].y, thr[0], thr[1]);
  if constexpr (MINV && Q == 1)
    return sweep_any8_min(a[0].x, a[0].y, a[1].x, a[1].y, a[2].x, a[2].y, a[3].x, a[3].y, thr[0], thr[0]);
  return sweep_any8(a[0].x, a[0].y, a[1].x, a[1].y, a[2].x, a[2].y, a[3].x, a[3].y, thr[0 % Q], thr[0 % Q],
                    thr[1 % Q], thr[1 % Q], thr[2 % Q], thr[2 % Q], thr[3 % Q], thr[3 % Q]);
}

// Two queries against four keys (two key pairs) as sweep_group2<2, true>, also returning the
// minimum filter value of each query, m[s], so that the verify path can skip a whole query.
__device__ __forceinline__ bool sweep_group2_gated(const float4 *__restrict__ pairs, const float2 (&mx)[2],
                                                   const float2 (&my)[2], const float2 (&mz)[2],
                                                   const float (&thr)[2], float2 (&a)[4], float (&m)[2]) {
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const float4 A = pairs[2 * p], Bv = pairs[2 * p + 1];
    const float2 kx = make_float2(A.x, A.y), ky = make_float2(A.z, A.w);
    const float2 kz = make_float2(Bv.x, Bv.y), kw = make_float2(Bv.z, Bv.w);
#pragma unroll
    for (int s = 0; s < 2; ++s) a[p * 2 + s] = __ffma2_rn(mx[s], kx, __ffma2_rn(my[s], ky, __ffma2_rn(mz[s], kz, kw)));
  }
  return sweep_any8_min2(a[0].x, a[0].y, a[2].x, a[2].y, a[1].x, a[1].y, a[3].x, a[3].y, thr[0], thr[1], m[0], m[1]);
}

}  // namespace tk3d
