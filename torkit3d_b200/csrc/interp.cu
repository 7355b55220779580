// Three-neighbour feature interpolation (forward / backward) and the inverse-distance weights.
//
//   out[b,c,m] = (in[b,c,i0]*w0 + in[b,c,i1]*w1) + in[b,c,i2]*w2,   (i*, w*) = index/weight[b,m,:]
//
// Memory-bound: the [B,C,N2] output dominates.  A thread owns one query m, loads its three indices
// and weights once (the reference re-reads them for every channel) and walks the channels; lanes
// of a warp hold consecutive m, so stores coalesce along N2.
#include "rows.cuh"

namespace tk3d {

namespace {

constexpr int IP_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(IP_THREADS)
interp_fwd_direct_kernel(const T *__restrict__ in, const int64_t *__restrict__ index, const T *__restrict__ weight,
                         int64_t C, int64_t N1, int64_t N2, int64_t c_per_block, T *__restrict__ out,
                         int32_t *__restrict__ status) {
  const int64_t b = blockIdx.z;
  const int64_t m = (int64_t)blockIdx.x * IP_THREADS + threadIdx.x;
  if (m >= N2) return;
  const int64_t c0 = (int64_t)blockIdx.y * c_per_block;
  const int64_t c1 = (c0 + c_per_block < C) ? c0 + c_per_block : C;
  int64_t id[3];
  T w[3];
  bool bad = false;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    id[i] = index[(b * N2 + m) * 3 + i];
    w[i] = weight[(b * N2 + m) * 3 + i];
    if (id[i] < 0 || id[i] >= N1) {
      id[i] = 0;
      w[i] = (T)0;
      bad = true;
    }
  }
  if (bad && status) atomicOr(status, 1);
  if (N1 == 0) {
    for (int64_t c = c0; c < c1; ++c) out[(b * C + c) * N2 + m] = (T)0;
    return;
  }
  const T *src = in + (b * C + c0) * N1;
  T *dst = out + (b * C + c0) * N2 + m;
#pragma unroll 4
  for (int64_t c = c0; c < c1; ++c, src += N1, dst += N2) {
    T acc = __ldg(src + id[0]) * w[0];
    acc += __ldg(src + id[1]) * w[1];
    acc += __ldg(src + id[2]) * w[2];
    __stcs(dst, acc);
  }
}

template <typename T>
__global__ void __launch_bounds__(IP_THREADS)
interp_bwd_kernel(const T *__restrict__ gout, const int64_t *__restrict__ index, const T *__restrict__ weight,
                  int64_t C, int64_t N1, int64_t N2, int64_t c_per_block, T *__restrict__ gin,
                  int32_t *__restrict__ status) {
  const int64_t b = blockIdx.z;
  const int64_t m = (int64_t)blockIdx.x * IP_THREADS + threadIdx.x;
  if (m >= N2) return;
  const int64_t c0 = (int64_t)blockIdx.y * c_per_block;
  const int64_t c1 = (c0 + c_per_block < C) ? c0 + c_per_block : C;
  int64_t id[3];
  T w[3];
  bool bad = false;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    id[i] = index[(b * N2 + m) * 3 + i];
    w[i] = weight[(b * N2 + m) * 3 + i];
    if (id[i] < 0 || id[i] >= N1) {
      id[i] = -1;
      bad = true;
    }
  }
  if (bad && status) atomicOr(status, 1);
  const T *src = gout + (b * C + c0) * N2 + m;
  T *dst = gin + (b * C + c0) * N1;
#pragma unroll 4
  for (int64_t c = c0; c < c1; ++c, src += N2, dst += N1) {
    const T g = __ldcs(src);
#pragma unroll
    for (int i = 0; i < 3; ++i)
      if (id[i] >= 0) atomicAdd(dst + id[i], g * w[i]);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
three_nn_weight_kernel(const T *__restrict__ dist, int64_t rows, int k, T *__restrict__ weight) {
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
    T inv[8];
    T sum = (T)0;
    for (int i = 0; i < k; ++i) {
      T d = dist[r * k + i];
      if (d < (T)1e-10) d = (T)1e-10;
      inv[i] = (T)1 / d;
      sum += inv[i];
    }
    for (int i = 0; i < k; ++i) weight[r * k + i] = inv[i] / sum;
  }
}

int64_t channels_per_block(int64_t tiles, int64_t B, int64_t C, int mult = 8) {
  const int64_t want = (int64_t)sm_count() * mult;
  int64_t groups = (want + tiles * B - 1) / (tiles * B);
  if (groups < 1) groups = 1;
  if (groups > C) groups = C;
  return (C + groups - 1) / groups;
}

template <typename T>
int interp_fwd_t(const T *in, const int64_t *index, const T *weight, int64_t B, int64_t C, int64_t N1, int64_t N2,
                 T *out, int32_t *status, cudaStream_t st) {
  const int64_t tiles = (N2 + IP_THREADS - 1) / IP_THREADS;
  const int64_t cpb = channels_per_block(tiles, B, C);
  const int64_t groups = (C + cpb - 1) / cpb;
  TK3D_REQUIRE(tiles < (1LL << 31) && groups <= 65535 && B <= 65535, TK3D_ERR_SHAPE, "interpolate: grid too large");
  dim3 grid((unsigned)tiles, (unsigned)groups, (unsigned)B);
  interp_fwd_direct_kernel<T><<<grid, IP_THREADS, 0, st>>>(in, index, weight, C, N1, N2, cpb, out, status);
  return check_launch("interp_fwd_direct_kernel");
}

template <typename T>
int interp_bwd_t(const T *gout, const int64_t *index, const T *weight, int64_t B, int64_t C, int64_t N1, int64_t N2,
                 T *gin, int32_t *status, cudaStream_t st) {
  TK3D_CUDA(cudaMemsetAsync(gin, 0, sizeof(T) * (size_t)(B * C * N1), st));
  if (N2 == 0) return TK3D_OK;
  const int64_t tiles = (N2 + IP_THREADS - 1) / IP_THREADS;
  // many small blocks: the atomics of a block that walks 13 channels arrive in bursts per row, and a
  // grid of little more than one wave has a tail (float64, 8 x 128 x 1024 <- 4096: 0.085 -> 0.069 ms)
  const int64_t cpb = channels_per_block(tiles, B, C, 128);
  const int64_t groups = (C + cpb - 1) / cpb;
  TK3D_REQUIRE(tiles < (1LL << 31) && groups <= 65535 && B <= 65535, TK3D_ERR_SHAPE, "interpolate: grid too large");
  dim3 grid((unsigned)tiles, (unsigned)groups, (unsigned)B);
  interp_bwd_kernel<T><<<grid, IP_THREADS, 0, st>>>(gout, index, weight, C, N1, N2, cpb, gin, status);
  return check_launch("interp_bwd_kernel");
}

int check_interp_args(const char *what, int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K, int dtype) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "%s: dtype %d", what, dtype);
  TK3D_REQUIRE(B >= 0 && C >= 0 && N1 >= 0 && N2 >= 0, TK3D_ERR_SHAPE, "%s: negative size", what);
  TK3D_REQUIRE(K == 3, TK3D_ERR_K, "%s: only k=3 is supported (got %lld)", what, (long long)K);
  TK3D_REQUIRE(N1 < (1LL << 31), TK3D_ERR_SHAPE, "%s: N1 limited to 2^31-1", what);
  return TK3D_OK;
}

}  // namespace
}  // namespace tk3d

using namespace tk3d;

extern "C" size_t tk3d_interp_fwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int dtype) {
  if (dtype != TK3D_F32 || B <= 0 || C <= 0 || N1 <= 0 || N2 <= 0 || B > 65535) return 0;
  return rows_profitable(C, N1, N2, 3) ? rows_scratch_bytes(B, C, N1) : 0;
}

extern "C" int tk3d_interp_fwd(const void *in, const int64_t *index, const void *weight, int64_t B, int64_t C,
                               int64_t N1, int64_t N2, int64_t K, void *out, int32_t *status, void *scratch,
                               size_t scratch_bytes, int dtype, void *stream) {
  TK3D_RANGE("tk3d_interp_fwd");
  int rc = check_interp_args("interp_fwd", B, C, N1, N2, K, dtype);
  if (rc) return rc;
  if (B * C * N2 == 0) return TK3D_OK;
  TK3D_REQUIRE(index && weight && out && (in || N1 == 0), TK3D_ERR_NULL, "interp_fwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F32) {
    const size_t want = tk3d_interp_fwd_scratch_bytes(B, C, N1, N2, dtype);
    if (want != 0 && scratch != nullptr && scratch_bytes >= want)
      return gather_rows<3>((const float *)in, index, (const float *)weight, B, C, N1, N2, (float *)out, status,
                            (float *)scratch, st);
    return interp_fwd_t<float>((const float *)in, index, (const float *)weight, B, C, N1, N2, (float *)out, status, st);
  }
  return interp_fwd_t<double>((const double *)in, index, (const double *)weight, B, C, N1, N2, (double *)out, status,
                              st);
}

extern "C" int tk3d_feature_rows(const void *feature, int64_t B, int64_t C, int64_t N, void *rows, int dtype,
                                 void *stream) {
  TK3D_RANGE("tk3d_feature_rows");
  TK3D_REQUIRE(dtype == TK3D_F32, TK3D_ERR_DTYPE, "feature_rows: float32 only (dtype %d)", dtype);
  TK3D_REQUIRE(B >= 0 && C >= 0 && N >= 0, TK3D_ERR_SHAPE, "feature_rows: negative size");
  if (B * C * N == 0) return TK3D_OK;
  TK3D_REQUIRE(feature && rows, TK3D_ERR_NULL, "feature_rows: a pointer is NULL");
  TK3D_REQUIRE(B <= 65535 && (C + 31) / 32 <= 65535, TK3D_ERR_SHAPE, "feature_rows: size too large");
  return transpose_bcn((const float *)feature, (float *)rows, B, C, N, (cudaStream_t)stream);
}

extern "C" int tk3d_interp_fwd_rows(const void *rows, const void *index, int index_dtype, const void *weight, int64_t B,
                                    int64_t C, int64_t N1, int64_t N2, int64_t K, void *out, int32_t *status,
                                    int dtype, void *stream) {
  TK3D_RANGE("tk3d_interp_fwd_rows");
  int rc = check_interp_args("interp_fwd_rows", B, C, N1, N2, K, dtype);
  if (rc) return rc;
  TK3D_REQUIRE(dtype == TK3D_F32, TK3D_ERR_DTYPE, "interp_fwd_rows: float32 only (dtype %d)", dtype);
  TK3D_REQUIRE(index_dtype == TK3D_I64 || index_dtype == TK3D_I32, TK3D_ERR_DTYPE, "interp_fwd_rows: index_dtype %d",
               index_dtype);
  TK3D_REQUIRE(C <= ROWS_MAX_C && B <= 65535, TK3D_ERR_SHAPE, "interp_fwd_rows: C <= %d and B <= 65535 required",
               ROWS_MAX_C);
  if (B * C * N2 == 0) return TK3D_OK;
  TK3D_REQUIRE(index && weight && out && (rows || N1 == 0), TK3D_ERR_NULL, "interp_fwd_rows: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (index_dtype == TK3D_I32)
    return gather_from_rows<3, int32_t>((const float *)rows, (const int32_t *)index, (const float *)weight, B, C, N1,
                                        N2, (float *)out, status, st);
  return gather_from_rows<3, int64_t>((const float *)rows, (const int64_t *)index, (const float *)weight, B, C, N1, N2,
                                      (float *)out, status, st);
}

extern "C" size_t tk3d_interp_bwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int dtype) {
  if (dtype != TK3D_F32 || C % 4 != 0 || N2 % 4 != 0 || (N1 + 31) / 32 > 65535) return 0;
  return tk3d_interp_fwd_scratch_bytes(B, C, N1, N2, dtype);
}

extern "C" int tk3d_interp_bwd(const void *gout, const int64_t *index, const void *weight, int64_t B, int64_t C,
                               int64_t N1, int64_t N2, int64_t K, void *gin, int32_t *status, void *scratch,
                               size_t scratch_bytes, int dtype, void *stream) {
  TK3D_RANGE("tk3d_interp_bwd");
  int rc = check_interp_args("interp_bwd", B, C, N1, N2, K, dtype);
  if (rc) return rc;
  if (B * C * N1 == 0) return TK3D_OK;
  TK3D_REQUIRE(gin && (N2 == 0 || (index && weight && gout)), TK3D_ERR_NULL, "interp_bwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F32) {
    const size_t want = tk3d_interp_bwd_scratch_bytes(B, C, N1, N2, dtype);
    if (want != 0 && scratch != nullptr && scratch_bytes >= want && rows_vec_ok(C, N2, gout, scratch))
      return scatter_rows<3>((const float *)gout, index, (const float *)weight, B, C, N1, N2, (float *)gin, status,
                             (float *)scratch, st);
    return interp_bwd_t<float>((const float *)gout, index, (const float *)weight, B, C, N1, N2, (float *)gin, status,
                               st);
  }
  return interp_bwd_t<double>((const double *)gout, index, (const double *)weight, B, C, N1, N2, (double *)gin,
                              status, st);
}

extern "C" int tk3d_three_nn_weight(const void *distance, int64_t rows, int64_t k, void *weight, int dtype,
                                    void *stream) {
  TK3D_RANGE("tk3d_three_nn_weight");
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "three_nn_weight: dtype %d", dtype);
  TK3D_REQUIRE(rows >= 0, TK3D_ERR_SHAPE, "three_nn_weight: negative size");
  TK3D_REQUIRE(k >= 1 && k <= 8, TK3D_ERR_K, "three_nn_weight: k must be in [1,8] (got %lld)", (long long)k);
  if (rows == 0) return TK3D_OK;
  TK3D_REQUIRE(distance && weight, TK3D_ERR_NULL, "three_nn_weight: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t want = (rows + 255) / 256, cap = (int64_t)sm_count() * 16;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  if (dtype == TK3D_F32)
    three_nn_weight_kernel<float><<<grid, 256, 0, st>>>((const float *)distance, rows, (int)k, (float *)weight);
  else
    three_nn_weight_kernel<double><<<grid, 256, 0, st>>>((const double *)distance, rows, (int)k, (double *)weight);
  return check_launch("three_nn_weight_kernel");
}

// ---------------------------------------------------------------------------------------------
// Fused feature interpolation: three nearest keys + inverse-distance weights + weighted gather.
namespace tk3d {

int three_nn_fused_f32(const float *query, const float *key, int64_t B, int64_t N1, int64_t N2, int channel_first,
                       float eps, float *weight, int32_t *index32, cudaStream_t st);

namespace {

// Backward without the row path: one thread per gradient element, 32-bit indices.
__global__ void __launch_bounds__(256)
interp32_bwd_kernel(const float *__restrict__ gout, const int32_t *__restrict__ index32,
                    const float *__restrict__ weight, int64_t B, int C, int64_t Nk, int64_t Nq,
                    float *__restrict__ gfeat, int32_t *__restrict__ status) {
  const int64_t total = B * C * Nq;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t q = t % Nq;
    const int64_t bc = t / Nq;
    const int64_t b = bc / C;
    const float g = gout[t];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int id = index32[(b * Nq + q) * 3 + i];
      if (id < 0 || id >= Nk) {
        if (status) atomicOr(status, 1);
        continue;
      }
      atomicAdd(gfeat + bc * Nk + id, g * weight[(b * Nq + q) * 3 + i]);
    }
  }
}

bool fused_interp_shape_ok(int64_t B, int64_t C, int64_t Nq, int64_t Nk) {
  return B >= 0 && B <= 65535 && C >= 0 && C <= ROWS_MAX_C && Nq >= 0 && Nq < (1LL << 30) && Nk >= 3 &&
         Nk < (1LL << 30);
}

}  // namespace
}  // namespace tk3d

extern "C" size_t tk3d_three_nn_interp_scratch_bytes(int64_t B, int64_t C, int64_t Nq, int64_t Nk, int dtype) {
  if (dtype != TK3D_F32 || !fused_interp_shape_ok(B, C, Nq, Nk) || B * C == 0) return 0;
  return rows_scratch_bytes(B, C, Nk);
}

extern "C" int tk3d_three_nn_interp_fwd(const void *query_xyz, const void *key_xyz, const void *key_feature,
                                        int64_t B, int64_t C, int64_t Nq, int64_t Nk, int xyz_channel_first,
                                        float eps, void *out, int32_t *index32, void *weight, int32_t *status,
                                        void *scratch, size_t scratch_bytes, int dtype, void *stream) {
  TK3D_RANGE("tk3d_three_nn_interp_fwd");
  TK3D_REQUIRE(dtype == TK3D_F32, TK3D_ERR_DTYPE, "three_nn_interp_fwd: only fp32 has a fused path (dtype %d)", dtype);
  TK3D_REQUIRE(B >= 0 && C >= 0 && Nq >= 0 && Nk >= 0, TK3D_ERR_SHAPE, "three_nn_interp_fwd: negative size");
  TK3D_REQUIRE(Nk >= 3, TK3D_ERR_K, "three_nn_interp_fwd: needs at least 3 key points (got %lld)", (long long)Nk);
  TK3D_REQUIRE(fused_interp_shape_ok(B, C, Nq, Nk), TK3D_ERR_SHAPE,
               "three_nn_interp_fwd: unsupported shape B=%lld C=%lld Nq=%lld Nk=%lld (C <= %d)", (long long)B,
               (long long)C, (long long)Nq, (long long)Nk, ROWS_MAX_C);
  if (B * Nq == 0) return TK3D_OK;
  TK3D_REQUIRE(query_xyz && key_xyz && index32 && weight && (C == 0 || (key_feature && out)), TK3D_ERR_NULL,
               "three_nn_interp_fwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  int rc = three_nn_fused_f32((const float *)query_xyz, (const float *)key_xyz, B, Nq, Nk, xyz_channel_first, eps,
                              (float *)weight, index32, st);
  if (rc || C == 0) return rc;
  const size_t want = rows_scratch_bytes(B, C, Nk);
  TK3D_REQUIRE(scratch != nullptr && scratch_bytes >= want, TK3D_ERR_SCRATCH,
               "three_nn_interp_fwd: scratch of %zu bytes required (got %zu)", want, scratch ? scratch_bytes : (size_t)0);
  return gather_rows<3, int32_t>((const float *)key_feature, index32, (const float *)weight, B, C, Nk, Nq,
                                 (float *)out, status, (float *)scratch, st);
}

extern "C" int tk3d_three_nn_interp_bwd(const void *gout, const int32_t *index32, const void *weight, int64_t B,
                                        int64_t C, int64_t Nq, int64_t Nk, void *gfeature, int32_t *status,
                                        void *scratch, size_t scratch_bytes, int dtype, void *stream) {
  TK3D_RANGE("tk3d_three_nn_interp_bwd");
  TK3D_REQUIRE(dtype == TK3D_F32, TK3D_ERR_DTYPE, "three_nn_interp_bwd: only fp32 has a fused path (dtype %d)", dtype);
  TK3D_REQUIRE(fused_interp_shape_ok(B, C, Nq, Nk), TK3D_ERR_SHAPE, "three_nn_interp_bwd: unsupported shape");
  if (B * C * Nk == 0) return TK3D_OK;
  TK3D_REQUIRE(gfeature && (Nq == 0 || (gout && index32 && weight)), TK3D_ERR_NULL,
               "three_nn_interp_bwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = C % 4 == 0 && Nq % 4 == 0 && (Nk + 31) / 32 <= 65535 && scratch != nullptr &&
                   scratch_bytes >= rows_scratch_bytes(B, C, Nk) && rows_vec_ok(C, Nq, gout, scratch);
  if (vec) {
    TK3D_CUDA(cudaMemsetAsync(scratch, 0, rows_scratch_bytes(B, C, Nk), st));
    if (Nq > 0) {
      const size_t smem = (size_t)C * ROWS_TE * sizeof(float);
      if (smem > 48 * 1024)
        TK3D_CUDA(raise_smem_limit((const void *)scatter_rows_vec4_kernel<3, int32_t>, (int)smem));
      dim3 grid((unsigned)((Nq + ROWS_TE - 1) / ROWS_TE), (unsigned)B);
      scatter_rows_vec4_kernel<3, int32_t><<<grid, ROWS_THREADS, smem, st>>>(
          (const float *)gout, index32, (const float *)weight, (int)C, Nk, Nq, C * Nq, (float *)scratch, status);
      int rc = check_launch("scatter_rows_vec4_kernel");
      if (rc) return rc;
    }
    return transpose_bcn((const float *)scratch, (float *)gfeature, B, Nk, C, st);
  }
  TK3D_CUDA(cudaMemsetAsync(gfeature, 0, sizeof(float) * (size_t)(B * C * Nk), st));
  if (Nq == 0) return TK3D_OK;
  const int64_t blocks = (B * C * Nq + 255) / 256, cap = (int64_t)sm_count() * 32;
  interp32_bwd_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(
      (const float *)gout, index32, (const float *)weight, B, (int)C, Nk, Nq, (float *)gfeature, status);
  return check_launch("interp32_bwd_kernel");
}

TK3D_BOUNDS_TU(interp)
