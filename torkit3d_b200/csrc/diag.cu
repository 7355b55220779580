// Diagnostics: a dependent-chain FFMA kernel that measures the FP32 fused-multiply-add rate the
// device sustains, i.e. the roofline the O(N*M) distance kernels are reported against.
#include "tk3d_common.cuh"

namespace tk3d {
namespace {

__global__ void __launch_bounds__(256) ffma_peak_kernel(int64_t iters, float seed, float *sink) {
  // 8 independent chains per thread keep the FMA pipe full at any occupancy used here.
  float a0 = seed + threadIdx.x, a1 = a0 + 1.f, a2 = a0 + 2.f, a3 = a0 + 3.f;
  float a4 = a0 + 4.f, a5 = a0 + 5.f, a6 = a0 + 6.f, a7 = a0 + 7.f;
  const float m = 0.999f, c = 0.001f;
  for (int64_t i = 0; i < iters; ++i) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      a0 = fmaf(a0, m, c);
      a1 = fmaf(a1, m, c);
      a2 = fmaf(a2, m, c);
      a3 = fmaf(a3, m, c);
      a4 = fmaf(a4, m, c);
      a5 = fmaf(a5, m, c);
      a6 = fmaf(a6, m, c);
      a7 = fmaf(a7, m, c);
    }
  }
  const float s = ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
  if (s == 123456.789f) *sink = s;  // never true in practice; keeps the chains alive
}

}  // namespace
}  // namespace tk3d

using namespace tk3d;

extern "C" int tk3d_diag_ffma(int64_t iters, float *sink, double *flop, void *stream) {
  TK3D_RANGE("tk3d_diag_ffma");
  TK3D_REQUIRE(iters > 0, TK3D_ERR_SHAPE, "diag_ffma: iters must be positive");
  TK3D_REQUIRE(sink != nullptr, TK3D_ERR_NULL, "diag_ffma: sink is NULL");
  const int blocks = sm_count() * 8;
  ffma_peak_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(iters, 1.0f, sink);
  if (flop) *flop = (double)blocks * 256.0 * (double)iters * 64.0 * 2.0;
  return check_launch("ffma_peak_kernel");
}

TK3D_BOUNDS_TU(diag)
