// Chamfer distance: nearest neighbour in both directions (forward) and the gradients w.r.t. both
// clouds (backward).
#include "tk3d_common.cuh"

namespace tk3d {

// ---------------------------------------------------------------------------------------------
// Generic forward (any floating type): one query per thread, 256-point key tiles in shared memory
// as structure-of-arrays so that every lane reads the same word (broadcast).
// Both directions run in one launch: block ids [0, blocks1) sweep cloud 2 for the points of cloud 1,
// the remaining ids do the opposite direction.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
chamfer_fwd_generic_kernel(const T *__restrict__ xyz1, const T *__restrict__ xyz2, int64_t B, int64_t N1,
                           int64_t N2, T *__restrict__ dist1, int64_t *__restrict__ idx1, T *__restrict__ dist2,
                           int64_t *__restrict__ idx2, double *__restrict__ sums, int64_t blocks1,
                           int64_t blocks_total, XyzLayout l1, XyzLayout l2) {
  constexpr int TILE = 256;
  __shared__ T sx[TILE], sy[TILE], sz[TILE];
  __shared__ double ssum[8];
  const int tid = threadIdx.x;

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int dir = blk >= blocks1;
    const int64_t id = dir ? blk - blocks1 : blk;
    const T *qpts = dir ? xyz2 : xyz1;
    const T *rpts = dir ? xyz1 : xyz2;
    const int64_t nq = dir ? N2 : N1;
    const int64_t nr = dir ? N1 : N2;
    const XyzLayout lq = dir ? l2 : l1, lr = dir ? l1 : l2;
    T *dist = dir ? dist2 : dist1;
    int64_t *idx = dir ? idx2 : idx1;
    const int64_t chunks = (nq + TILE - 1) / TILE;
    const int64_t b = id / chunks;
    const int64_t i = (id % chunks) * TILE + tid;
    const bool valid = i < nq;

    T qx = 0, qy = 0, qz = 0;
    if (valid) load_xyz(qpts + b * nq * 3, i, lq, qx, qy, qz);
    T best = Exact<T>::inf();
    int64_t arg = -1;
    const T *rb = rpts + b * nr * 3;
    for (int64_t t0 = 0; t0 < nr; t0 += TILE) {
      const int64_t j = t0 + tid;
      if (j < nr) load_xyz(rb, j, lr, sx[tid], sy[tid], sz[tid]);
      __syncthreads();
      const int lim = (int)((nr - t0) < TILE ? (nr - t0) : TILE);
      for (int u = 0; u < lim; ++u) {
        T d = sqdist<T>(sx[u], sy[u], sz[u], qx, qy, qz);
        if (d < best) {
          best = d;
          arg = t0 + u;
        }
      }
      __syncthreads();
    }
    if (valid) {
      dist[b * nq + i] = best;
      idx[b * nq + i] = arg;
    }
    if (sums != nullptr) {
      double v = warp_sum(valid ? (double)best : 0.0);
      if ((tid & 31) == 0) ssum[tid >> 5] = v;
      __syncthreads();
      if (tid == 0) {
        double s = 0;
#pragma unroll
        for (int w = 0; w < TILE / 32; ++w) s += ssum[w];
        atomicAdd(sums + dir, s);
      }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Backward.  Pass A writes each point's own term with plain stores (no zero-fill, no atomics):
//   grad_a[i] = 2 g[i] (a_i - b_idx[i]).
// Pass B scatters the opposite-sign term onto the matched point of the other cloud with atomics.
// Stream order between the two launches guarantees A's stores land before B's atomics.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
chamfer_bwd_own_kernel(const T *__restrict__ g1, const T *__restrict__ g2, const T *__restrict__ xyz1,
                       const T *__restrict__ xyz2, const int64_t *__restrict__ idx1,
                       const int64_t *__restrict__ idx2, int64_t B, int64_t N1, int64_t N2, T *__restrict__ grad1,
                       T *__restrict__ grad2, int gstride, T scale1, T scale2, XyzLayout l1, XyzLayout l2) {
  const int64_t tot1 = B * N1, total = B * (N1 + N2);
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int dir = t >= tot1;
    const int64_t lin = dir ? t - tot1 : t;
    const int64_t na = dir ? N2 : N1, nb = dir ? N1 : N2;
    const XyzLayout la = dir ? l2 : l1, lb = dir ? l1 : l2;
    const T *a = dir ? xyz2 : xyz1;
    const T *bb = dir ? xyz1 : xyz2;
    const int64_t b = lin / na, i = lin - b * na;
    const int64_t j = (dir ? idx2 : idx1)[lin];
    T *ga = (dir ? grad2 : grad1) + b * na * 3 + i * la.ps;  // gradients share their cloud's layout
    if (j < 0 || j >= nb) {
      ga[0] = 0;
      ga[la.cs] = 0;
      ga[2 * (int64_t)la.cs] = 0;
      continue;
    }
    // gstride 0: one upstream value for the whole cloud set; scale is 1 for per-point gradients
    const T g = (dir ? g2 : g1)[lin * gstride] * (dir ? scale2 : scale1) * (T)2;
    T px, py, pz, qx, qy, qz;
    load_xyz(a + b * na * 3, i, la, px, py, pz);
    load_xyz(bb + b * nb * 3, j, lb, qx, qy, qz);
    ga[0] = g * (px - qx);
    ga[la.cs] = g * (py - qy);
    ga[2 * (int64_t)la.cs] = g * (pz - qz);
  }
}

// Atomic add of a 3-vector to a row of an [.,3] array.  A row starts on an 8-byte boundary every
// other point, so two of the three floats always go out as one vector reduction (red.v2.f32).
__device__ __forceinline__ void red_add3(float *p, float a, float b, float c) {
  if ((reinterpret_cast<uintptr_t>(p) & 7) == 0) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(a), "f"(b) : "memory");
    atomicAdd(p + 2, c);
  } else {
    atomicAdd(p, a);
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p + 1), "f"(b), "f"(c) : "memory");
  }
}
__device__ __forceinline__ void red_add3(double *p, double a, double b, double c) {
  atomicAdd(p + 0, a);
  atomicAdd(p + 1, b);
  atomicAdd(p + 2, c);
}

template <typename T>
__global__ void __launch_bounds__(256)
chamfer_bwd_scatter_kernel(const T *__restrict__ g1, const T *__restrict__ g2, const T *__restrict__ xyz1,
                           const T *__restrict__ xyz2, const int64_t *__restrict__ idx1,
                           const int64_t *__restrict__ idx2, int64_t B, int64_t N1, int64_t N2, T *grad1, T *grad2,
                           int gstride, T scale1, T scale2, XyzLayout l1, XyzLayout l2) {
  const int64_t tot1 = B * N1, total = B * (N1 + N2);
  for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int dir = t >= tot1;
    const int64_t lin = dir ? t - tot1 : t;
    const int64_t na = dir ? N2 : N1, nb = dir ? N1 : N2;
    const XyzLayout la = dir ? l2 : l1, lb = dir ? l1 : l2;
    const T *a = dir ? xyz2 : xyz1;
    const T *bb = dir ? xyz1 : xyz2;
    const int64_t b = lin / na, i = lin - b * na;
    const int64_t j = (dir ? idx2 : idx1)[lin];
    if (j < 0 || j >= nb) continue;
    // gstride 0: one upstream value for the whole cloud set; scale is 1 for per-point gradients
    const T g = (dir ? g2 : g1)[lin * gstride] * (dir ? scale2 : scale1) * (T)2;
    T px, py, pz, qx, qy, qz;
    load_xyz(a + b * na * 3, i, la, px, py, pz);
    load_xyz(bb + b * nb * 3, j, lb, qx, qy, qz);
    T *gb = (dir ? grad1 : grad2) + b * nb * 3 + j * lb.ps;
    if (lb.cs == 1) {
      red_add3(gb, -(g * (px - qx)), -(g * (py - qy)), -(g * (pz - qz)));
    } else {
      atomicAdd(gb, -(g * (px - qx)));
      atomicAdd(gb + lb.cs, -(g * (py - qy)));
      atomicAdd(gb + 2 * (int64_t)lb.cs, -(g * (pz - qz)));
    }
  }
}

int chamfer_fwd_f32_fast(const float *xyz1, const float *xyz2, int64_t B, int64_t N1, int64_t N2, float *dist1,
                         int64_t *idx1, float *dist2, int64_t *idx2, double *sums, cudaStream_t st, XyzLayout l1,
                         XyzLayout l2);

template <typename T>
static int chamfer_fwd_generic(const T *xyz1, const T *xyz2, int64_t B, int64_t N1, int64_t N2, T *dist1,
                               int64_t *idx1, T *dist2, int64_t *idx2, double *sums, cudaStream_t st, XyzLayout l1,
                               XyzLayout l2) {
  const int64_t blocks1 = B * ((N1 + 255) / 256), blocks2 = B * ((N2 + 255) / 256);
  const int64_t total = blocks1 + blocks2;
  if (total == 0) return TK3D_OK;
  const int64_t cap = (int64_t)sm_count() * 64;
  const unsigned grid = (unsigned)(total < cap ? total : cap);
  chamfer_fwd_generic_kernel<T><<<grid, 256, 0, st>>>(xyz1, xyz2, B, N1, N2, dist1, idx1, dist2, idx2, sums,
                                                       blocks1, total, l1, l2);
  return check_launch("chamfer_fwd_generic_kernel");
}

template <typename T>
static int chamfer_bwd_t(const T *g1, const T *g2, const T *xyz1, const T *xyz2, const int64_t *idx1,
                         const int64_t *idx2, int64_t B, int64_t N1, int64_t N2, T *grad1, T *grad2,
                         cudaStream_t st, int channel_first, int gstride = 1, T scale1 = (T)1, T scale2 = (T)1) {
  const int64_t total = B * (N1 + N2);
  const XyzLayout l1 = xyz_layout(channel_first, N1), l2 = xyz_layout(channel_first, N2);
  if (total == 0) return TK3D_OK;
  const int64_t want = (total + 255) / 256, cap = (int64_t)sm_count() * 32;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  chamfer_bwd_own_kernel<T><<<grid, 256, 0, st>>>(g1, g2, xyz1, xyz2, idx1, idx2, B, N1, N2, grad1, grad2, gstride,
                                                  scale1, scale2, l1, l2);
  int rc = check_launch("chamfer_bwd_own_kernel");
  if (rc) return rc;
  chamfer_bwd_scatter_kernel<T><<<grid, 256, 0, st>>>(g1, g2, xyz1, xyz2, idx1, idx2, B, N1, N2, grad1, grad2,
                                                      gstride, scale1, scale2, l1, l2);
  return check_launch("chamfer_bwd_scatter_kernel");
}

// loss = sums[0] / count1 + sums[1] / count2, written as one element of type T
template <typename T>
__global__ void chamfer_mean_loss_kernel(const double *__restrict__ sums, double count1, double count2,
                                         T *__restrict__ loss) {
  if (threadIdx.x == 0 && blockIdx.x == 0) loss[0] = (T)(sums[0] / count1 + sums[1] / count2);
}

}  // namespace tk3d

using namespace tk3d;

extern "C" int tk3d_chamfer_mean_loss(const double *sums, double count1, double count2, void *loss, int dtype,
                                      void *stream) {
  TK3D_RANGE("tk3d_chamfer_mean_loss");
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "chamfer_mean_loss: dtype %d", dtype);
  TK3D_REQUIRE(sums && loss, TK3D_ERR_NULL, "chamfer_mean_loss: a pointer is NULL");
  TK3D_REQUIRE(count1 > 0 && count2 > 0, TK3D_ERR_SHAPE, "chamfer_mean_loss: counts must be positive");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F32)
    chamfer_mean_loss_kernel<float><<<1, 32, 0, st>>>(sums, count1, count2, (float *)loss);
  else
    chamfer_mean_loss_kernel<double><<<1, 32, 0, st>>>(sums, count1, count2, (double *)loss);
  return check_launch("chamfer_mean_loss_kernel");
}

static int chamfer_bwd_mean_impl(const void *grad_loss, double count1, double count2, const void *xyz1,
                                 const void *xyz2, const int64_t *idx1, const int64_t *idx2, int64_t B, int64_t N1,
                                 int64_t N2, int channel_first, void *grad1, void *grad2, int dtype, void *stream) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "chamfer_bwd_mean: dtype %d", dtype);
  TK3D_REQUIRE(B >= 0 && N1 >= 0 && N2 >= 0, TK3D_ERR_SHAPE, "chamfer_bwd_mean: negative size");
  TK3D_REQUIRE(count1 > 0 && count2 > 0, TK3D_ERR_SHAPE, "chamfer_bwd_mean: counts must be positive");
  TK3D_REQUIRE(grad_loss, TK3D_ERR_NULL, "chamfer_bwd_mean: grad_loss is NULL");
  TK3D_REQUIRE(B * N1 == 0 || (xyz1 && idx1 && grad1), TK3D_ERR_NULL, "chamfer_bwd_mean: a cloud-1 pointer is NULL");
  TK3D_REQUIRE(B * N2 == 0 || (xyz2 && idx2 && grad2), TK3D_ERR_NULL, "chamfer_bwd_mean: a cloud-2 pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F32)
    return chamfer_bwd_t<float>((const float *)grad_loss, (const float *)grad_loss, (const float *)xyz1,
                                (const float *)xyz2, idx1, idx2, B, N1, N2, (float *)grad1, (float *)grad2, st,
                                channel_first, 0, (float)(1.0 / count1), (float)(1.0 / count2));
  return chamfer_bwd_t<double>((const double *)grad_loss, (const double *)grad_loss, (const double *)xyz1,
                               (const double *)xyz2, idx1, idx2, B, N1, N2, (double *)grad1, (double *)grad2, st,
                               channel_first, 0, 1.0 / count1, 1.0 / count2);
}

extern "C" int tk3d_chamfer_bwd_mean(const void *grad_loss, double count1, double count2, const void *xyz1,
                                     const void *xyz2, const int64_t *idx1, const int64_t *idx2, int64_t B,
                                     int64_t N1, int64_t N2, void *grad1, void *grad2, int dtype, void *stream) {
  TK3D_RANGE("tk3d_chamfer_bwd_mean");
  return chamfer_bwd_mean_impl(grad_loss, count1, count2, xyz1, xyz2, idx1, idx2, B, N1, N2, 0, grad1, grad2, dtype,
                               stream);
}

extern "C" int tk3d_chamfer_bwd_mean_layout(const void *grad_loss, double count1, double count2, const void *xyz1,
                                            const void *xyz2, const int64_t *idx1, const int64_t *idx2, int64_t B,
                                            int64_t N1, int64_t N2, int xyz_channel_first, void *grad1, void *grad2,
                                            int dtype, void *stream) {
  TK3D_RANGE("tk3d_chamfer_bwd_mean_layout");
  return chamfer_bwd_mean_impl(grad_loss, count1, count2, xyz1, xyz2, idx1, idx2, B, N1, N2, xyz_channel_first != 0,
                               grad1, grad2, dtype, stream);
}

namespace tk3d {
const char *chamfer_fwd_f32_kernel_name(int64_t B, int64_t N1, int64_t N2);
}

extern "C" const char *tk3d_chamfer_fwd_kernel_name(int64_t B, int64_t N1, int64_t N2, int dtype) {
  if (dtype != TK3D_F32) return "chamfer_fwd_generic_kernel";
  return chamfer_fwd_f32_kernel_name(B < 0 ? 0 : B, N1 < 0 ? 0 : N1, N2 < 0 ? 0 : N2);
}

static int chamfer_fwd_impl(const void *xyz1, const void *xyz2, int64_t B, int64_t N1, int64_t N2, int channel_first,
                            void *dist1, int64_t *idx1, void *dist2, int64_t *idx2, double *sums, int dtype,
                            void *stream) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "chamfer_fwd: dtype %d", dtype);
  TK3D_REQUIRE(B >= 0 && N1 >= 0 && N2 >= 0, TK3D_ERR_SHAPE, "chamfer_fwd: negative size (B=%lld N1=%lld N2=%lld)",
               (long long)B, (long long)N1, (long long)N2);
  TK3D_REQUIRE(N1 < (1LL << 31) && N2 < (1LL << 31), TK3D_ERR_SHAPE, "chamfer_fwd: clouds limited to 2^31-1 points");
  TK3D_REQUIRE(B * N1 == 0 || (xyz1 && dist1 && idx1), TK3D_ERR_NULL, "chamfer_fwd: xyz1/dist1/idx1 is NULL");
  TK3D_REQUIRE(B * N2 == 0 || (xyz2 && dist2 && idx2), TK3D_ERR_NULL, "chamfer_fwd: xyz2/dist2/idx2 is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (sums) TK3D_CUDA(cudaMemsetAsync(sums, 0, 2 * sizeof(double), st));
  const XyzLayout l1 = xyz_layout(channel_first, N1), l2 = xyz_layout(channel_first, N2);
  if (dtype == TK3D_F32)
    return chamfer_fwd_f32_fast((const float *)xyz1, (const float *)xyz2, B, N1, N2, (float *)dist1, idx1,
                                (float *)dist2, idx2, sums, st, l1, l2);
  return chamfer_fwd_generic<double>((const double *)xyz1, (const double *)xyz2, B, N1, N2, (double *)dist1, idx1,
                                     (double *)dist2, idx2, sums, st, l1, l2);
}

extern "C" int tk3d_chamfer_fwd(const void *xyz1, const void *xyz2, int64_t B, int64_t N1, int64_t N2, void *dist1,
                                int64_t *idx1, void *dist2, int64_t *idx2, double *sums, int dtype, void *stream) {
  TK3D_RANGE("tk3d_chamfer_fwd");
  return chamfer_fwd_impl(xyz1, xyz2, B, N1, N2, 0, dist1, idx1, dist2, idx2, sums, dtype, stream);
}

extern "C" int tk3d_chamfer_fwd_layout(const void *xyz1, const void *xyz2, int64_t B, int64_t N1, int64_t N2,
                                       int xyz_channel_first, void *dist1, int64_t *idx1, void *dist2, int64_t *idx2,
                                       double *sums, int dtype, void *stream) {
  TK3D_RANGE("tk3d_chamfer_fwd_layout");
  return chamfer_fwd_impl(xyz1, xyz2, B, N1, N2, xyz_channel_first != 0, dist1, idx1, dist2, idx2, sums, dtype,
                          stream);
}

static int chamfer_bwd_impl(const void *g1, const void *g2, const void *xyz1, const void *xyz2, const int64_t *idx1,
                            const int64_t *idx2, int64_t B, int64_t N1, int64_t N2, int channel_first, void *grad1,
                            void *grad2, int dtype, void *stream) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "chamfer_bwd: dtype %d", dtype);
  TK3D_REQUIRE(B >= 0 && N1 >= 0 && N2 >= 0, TK3D_ERR_SHAPE, "chamfer_bwd: negative size");
  TK3D_REQUIRE(B * N1 == 0 || (g1 && xyz1 && idx1 && grad1), TK3D_ERR_NULL, "chamfer_bwd: a cloud-1 pointer is NULL");
  TK3D_REQUIRE(B * N2 == 0 || (g2 && xyz2 && idx2 && grad2), TK3D_ERR_NULL, "chamfer_bwd: a cloud-2 pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F32)
    return chamfer_bwd_t<float>((const float *)g1, (const float *)g2, (const float *)xyz1, (const float *)xyz2, idx1,
                                idx2, B, N1, N2, (float *)grad1, (float *)grad2, st, channel_first);
  return chamfer_bwd_t<double>((const double *)g1, (const double *)g2, (const double *)xyz1, (const double *)xyz2,
                               idx1, idx2, B, N1, N2, (double *)grad1, (double *)grad2, st, channel_first);
}

extern "C" int tk3d_chamfer_bwd(const void *g1, const void *g2, const void *xyz1, const void *xyz2,
                                const int64_t *idx1, const int64_t *idx2, int64_t B, int64_t N1, int64_t N2,
                                void *grad1, void *grad2, int dtype, void *stream) {
  TK3D_RANGE("tk3d_chamfer_bwd");
  return chamfer_bwd_impl(g1, g2, xyz1, xyz2, idx1, idx2, B, N1, N2, 0, grad1, grad2, dtype, stream);
}

extern "C" int tk3d_chamfer_bwd_layout(const void *g1, const void *g2, const void *xyz1, const void *xyz2,
                                       const int64_t *idx1, const int64_t *idx2, int64_t B, int64_t N1, int64_t N2,
                                       int xyz_channel_first, void *grad1, void *grad2, int dtype, void *stream) {
  TK3D_RANGE("tk3d_chamfer_bwd_layout");
  return chamfer_bwd_impl(g1, g2, xyz1, xyz2, idx1, idx2, B, N1, N2, xyz_channel_first != 0, grad1, grad2, dtype,
                          stream);
}

TK3D_BOUNDS_TU(chamfer)
