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

// Raise a kernel's dynamic shared-memory limit on the current device, once per (kernel, device).
cudaError_t raise_smem_limit(const void *func, int bytes);

// NVTX range spanning one entry point of the C ABI (host side: argument checks and launches), so
// that a timeline shows which operator enqueued which kernels.  NVTX binds lazily: without a
// profiler attached a push / pop is a load and a branch.
void nvtx_push(const char *name);
void nvtx_pop();
struct NvtxRange {
  explicit NvtxRange(const char *name) { nvtx_push(name); }
  ~NvtxRange() { nvtx_pop(); }
  NvtxRange(const NvtxRange &) = delete;
  NvtxRange &operator=(const NvtxRange &) = delete;
};
#define TK3D_RANGE(name) ::tk3d::NvtxRange tk3d_nvtx_range_(name)

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

// ---- coordinate layout and index type of the operator entry points --------------------------
// A batch of clouds is [B,N,3] (ps = 3, cs = 1: the reference's operator layout) or [B,3,N]
// (ps = 1, cs = N: the layout its layers pass around).  Cloud b starts at base + b*3*N in both;
// coordinate c of its point j is cloud[j*ps + c*cs].
//
// Range-checked build (-DTK3D_BOUNDS, libtk3d_b200_bounds.so): every coordinate load and every
// index-tensor access made through the helpers below is checked against the extent of its tensor;
// a violation is counted (one counter per translation unit, summed by tk3d_bounds_violations())
// and the access is redirected to element 0, so a logic error shows up as a number instead of a
// fault.  The regular build carries none of this.
#ifdef TK3D_BOUNDS
static __device__ unsigned long long tk3d_oob_count;
__device__ __forceinline__ int64_t tk3d_checked(int64_t i, int64_t n) {
  if (i < 0 || i >= n) {
    atomicAdd(&tk3d_oob_count, 1ull);
    return 0;
  }
  return i;
}
#define TK3D_BOUNDS_TU(tag)                                                   \
  extern "C" unsigned long long tk3d_bounds_count_##tag(void) {               \
    unsigned long long v = 0;                                                 \
    cudaMemcpyFromSymbol(&v, tk3d::tk3d_oob_count, sizeof(v));                \
    return v;                                                                 \
  }
#else
#define TK3D_BOUNDS_TU(tag)
#endif

struct XyzLayout {
  int ps, cs;
#ifdef TK3D_BOUNDS
  int n;  // points per cloud
#endif
};
inline XyzLayout xyz_layout(int channel_first, int64_t n) {
  XyzLayout l;
  l.ps = channel_first ? 1 : 3;
  l.cs = channel_first ? (int)n : 1;
#ifdef TK3D_BOUNDS
  l.n = (int)n;
#endif
  return l;
}
template <typename T>
__device__ __forceinline__ void load_xyz(const T *__restrict__ cloud, int64_t j, XyzLayout l, T &x, T &y, T &z) {
#ifdef TK3D_BOUNDS
  j = tk3d_checked(j, l.n);
#endif
  const T *p = cloud + j * l.ps;
  x = p[0];
  y = p[l.cs];
  z = p[2 * (int64_t)l.cs];
}

// Index tensors are int64 (the reference's type) or, as an opt-in of the *_layout entry points,
// int32 (half the bytes; every index fits, clouds are limited to 2^30 points).
struct IndexOut {
  void *p;
  int i32;
#ifdef TK3D_BOUNDS
  int64_t count;  // elements of the tensor
#endif
  __device__ __forceinline__ void put(int64_t off, int64_t v) const {
#ifdef TK3D_BOUNDS
    off = tk3d_checked(off, count);
#endif
    if (i32) static_cast<int32_t *>(p)[off] = (int32_t)v;
    else static_cast<int64_t *>(p)[off] = v;
  }
  __device__ __forceinline__ int64_t get(int64_t off) const {
#ifdef TK3D_BOUNDS
    off = tk3d_checked(off, count);
#endif
    return i32 ? (int64_t) static_cast<const int32_t *>(p)[off] : static_cast<const int64_t *>(p)[off];
  }
};
inline IndexOut index_out(void *p, int i32, int64_t count) {
  IndexOut o;
  o.p = p;
  o.i32 = i32;
#ifdef TK3D_BOUNDS
  o.count = count;
#else
  (void)count;
#endif
  return o;
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace tk3d
