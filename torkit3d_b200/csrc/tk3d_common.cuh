// Shared helpers of libtk3d_b200: error plumbing, exact (never fused) arithmetic, small reductions.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tk3d.h"

namespace tk3d {

// ---- error plumbing ------------------------------------------------------------------------
// The detailed message of the last failing call on this host thread.
char *last_error_buffer();
int fail(int code, const char *fmt, ...);

#define TK3D_REQUIRE(cond, code, ...)            \
  do {                                           \
    if (!(cond)) return ::tk3d::fail(code, __VA_ARGS__); \
  } while (0)

#define TK3D_CUDA(expr)                                                                          \
  do {                                                                                           \
    cudaError_t e__ = (expr);                                                                    \
    if (e__ != cudaSuccess)                                                                      \
      return ::tk3d::fail(TK3D_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));       \
  } while (0)

inline int check_launch(const char *what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(TK3D_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  return TK3D_OK;
}

// Number of SMs of the current device (cached per device id; read-only after first use).
int sm_count();

// ---- exact arithmetic ----------------------------------------------------------------------
// The round-to-nearest intrinsics are never contracted into a fused multiply-add by the compiler,
// which is what keeps index results bit-reproducible against a CPU evaluation.
template <typename T>
struct Exact;
template <>
struct Exact<float> {
  static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
  static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
  static __device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
  static __device__ __forceinline__ float inf() { return __int_as_float(0x7f800000); }
};
template <>
struct Exact<double> {
  static __device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
  static __device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
  static __device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
  static __device__ __forceinline__ double inf() { return __longlong_as_double(0x7ff0000000000000LL); }
};

// ((dx*dx + dy*dy) + dz*dz), d = ref - query.
template <typename T>
__device__ __forceinline__ T sqdist(T rx, T ry, T rz, T qx, T qy, T qz) {
  using E = Exact<T>;
  T dx = E::sub(rx, qx), dy = E::sub(ry, qy), dz = E::sub(rz, qz);
  return E::add(E::add(E::mul(dx, dx), E::mul(dy, dy)), E::mul(dz, dz));
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace tk3d
