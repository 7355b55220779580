// EdgeConv edge features (fp32 and fp64):
//     out[b, c,     n, k] = key_feature[b, c, index[b,n,k]] - query_feature[b, c, n]
//     out[b, C + c, n, k] = query_feature[b, c, n]                       (when include_query)
// i.e. group_points + broadcast subtraction + concatenation in one pass over the output, which is
// the only large tensor involved (2*C*N*K elements): the grouped features are never written
// un-centred and the concatenation is not a second copy.
//
// fp32 with C % 4 == 0 and (N*K) % 4 == 0 takes the row path of rows.cuh: key features transposed
// once into caller scratch [B,N2,C], rows fetched with 16-byte loads, channel-major output through
// the chunk-swizzled shared tile with 16-byte streaming stores.  Everything else takes a direct
// kernel (one thread per output entry, walking the channels).
#include "rows.cuh"

namespace tk3d {

namespace {

__global__ void __launch_bounds__(ROWS_THREADS)
edge_rows_vec4_kernel(const float *__restrict__ keyT, const float *__restrict__ qfeat,
                      const int64_t *__restrict__ index, int C, int64_t N2, int64_t N1, int K, int include_query,
                      float *__restrict__ out, int32_t *__restrict__ status) {
  extern __shared__ __align__(16) float tile[];  // [C][ROWS_TE], chunk-swizzled
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ql = lane & 7, el = lane >> 3;
  const int64_t b = blockIdx.y;
  const int64_t E = N1 * K;
  const int64_t e0 = (int64_t)blockIdx.x * ROWS_TE;
  const int n = (int)((E - e0) < ROWS_TE ? (E - e0) : ROWS_TE);  // multiple of 4
  const int L = C >> 2;

  // Four entries per warp and step, as in gather_rows_vec4_kernel: conflict-free scalar stores.
  const float4 *fb = reinterpret_cast<const float4 *>(keyT + b * N2 * C);
  bool bad = false;
  for (int g = warp; g < (n >> 2); g += ROWS_THREADS / 32) {
    int id[1];
    float w[1];
    rows_load_index<1, int64_t>(index, nullptr, b * E + e0 + 4 * g + el, N2, true, id, w, bad);
    const float4 *row = fb + (int64_t)(id[0] < 0 ? 0 : id[0]) * L;
#pragma unroll 4
    for (int q = ql; q < L; q += 8) {
      const float4 v = id[0] < 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : __ldg(row + q);
      float *dst = tile + (4 * q) * ROWS_TE + (((g ^ q) & (ROWS_TE / 4 - 1)) << 2) + el;
      dst[0] = v.x;
      dst[ROWS_TE] = v.y;
      dst[2 * ROWS_TE] = v.z;
      dst[3 * ROWS_TE] = v.w;
    }
  }
  if (bad && status) atomicOr(status, 1);
  __syncthreads();

  // item u = c * 16 + chunk: four consecutive entries of channel c; their query point is (e0+4ch+i)/K
  const int nchunks = n >> 2;
  const int ctot = include_query ? 2 * C : C;
  float *ob = out + b * ctot * E + e0;
  const float *qb = qfeat + b * C * N1;
  for (int u = tid; u < C * (ROWS_TE / 4); u += ROWS_THREADS) {
    const int c = u / ROWS_CH, ch = u % ROWS_CH;
    if (ch < nchunks) {
      float4 v = *reinterpret_cast<const float4 *>(tile + c * ROWS_TE + (((ch ^ (c >> 2)) & (ROWS_CH - 1)) << 2));
      // query point of each of the four entries: one 32-bit division, then a carry chain
      const unsigned eg = (unsigned)(e0 + 4 * ch);
      unsigned nq = eg / (unsigned)K;
      int r = (int)(eg - nq * (unsigned)K);
      const float *qp = qb + (int64_t)c * N1;
      float4 qv;
      qv.x = __ldg(qp + nq);
      if (++r == K) { r = 0; ++nq; }
      qv.y = __ldg(qp + nq);
      if (++r == K) { r = 0; ++nq; }
      qv.z = __ldg(qp + nq);
      if (++r == K) { r = 0; ++nq; }
      qv.w = __ldg(qp + nq);
      v.x = __fsub_rn(v.x, qv.x);
      v.y = __fsub_rn(v.y, qv.y);
      v.z = __fsub_rn(v.z, qv.z);
      v.w = __fsub_rn(v.w, qv.w);
      __stcs(reinterpret_cast<float4 *>(ob + (int64_t)c * E + 4 * ch), v);
      if (include_query) __stcs(reinterpret_cast<float4 *>(ob + (int64_t)(C + c) * E + 4 * ch), qv);
    }
  }
}

// Direct form: one thread per entry (b, n, k), walking the channels.
template <typename T>
__global__ void __launch_bounds__(256)
edge_direct_kernel(const T *__restrict__ key, const T *__restrict__ qfeat, const int64_t *__restrict__ index,
                   int64_t B, int64_t C, int64_t N2, int64_t N1, int64_t K, int include_query, T *__restrict__ out,
                   int32_t *__restrict__ status) {
  const int64_t E = N1 * K;
  const int64_t ctot = include_query ? 2 * C : C;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < B * E; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t b = t / E, e = t - b * E, n = e / K;
    int64_t id = index[t];
    if (id < 0 || id >= N2) {
      id = -1;
      if (status) atomicOr(status, 1);
    }
    const T *kb = key + b * C * N2;
    const T *qb = qfeat + b * C * N1 + n;
    T *ob = out + b * ctot * E + e;
    for (int64_t c = 0; c < C; ++c) {
      const T qv = qb[c * N1];
      const T kv = id < 0 ? (T)0 : kb[c * N2 + id];
      ob[c * E] = Exact<T>::sub(kv, qv);
      if (include_query) ob[(C + c) * E] = qv;
    }
  }
}

// grad_query[b,c,n] = sum_k (g[b,C+c,n,k] - g[b,c,n,k])   (second term only without include_query)
template <typename T>
__global__ void __launch_bounds__(256)
edge_bwd_query_kernel(const T *__restrict__ gout, int64_t B, int64_t C, int64_t N1, int64_t K, int include_query,
                      T *__restrict__ gq) {
  const int64_t E = N1 * K;
  const int64_t ctot = include_query ? 2 * C : C;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < B * C * N1;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = t % N1;
    const int64_t bc = t / N1;
    const int64_t b = bc / C, c = bc - b * C;
    const T *g0 = gout + (b * ctot + c) * E + n * K;
    const T *g1 = gout + (b * ctot + C + c) * E + n * K;
    T acc = 0;
    for (int64_t k = 0; k < K; ++k) acc += include_query ? g1[k] - g0[k] : -g0[k];
    gq[t] = acc;
  }
}

// grad_key without the row path: scalar atomics.
template <typename T>
__global__ void __launch_bounds__(256)
edge_bwd_key_kernel(const T *__restrict__ gout, const int64_t *__restrict__ index, int64_t B, int64_t C, int64_t N2,
                    int64_t E, int64_t gstride, T *__restrict__ gk, int32_t *__restrict__ status) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < B * C * E;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = t % E;
    const int64_t bc = t / E;
    const int64_t b = bc / C, c = bc - b * C;
    const int64_t id = index[b * E + e];
    if (id < 0 || id >= N2) {
      if (status) atomicOr(status, 1);
      continue;
    }
    atomicAdd(gk + bc * N2 + id, gout[b * gstride + c * E + e]);
  }
}

bool edge_shape_ok(int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K) {
  return B >= 0 && C >= 0 && N1 >= 0 && N2 >= 0 && K >= 0 && N2 < (1LL << 31) && N1 < (1LL << 31) && K < (1LL << 31);
}

template <typename T>
int edge_fwd_direct(const T *key, const T *q, const int64_t *index, int64_t B, int64_t C, int64_t N2, int64_t N1,
                    int64_t K, int include_query, T *out, int32_t *status, cudaStream_t st) {
  const int64_t blocks = (B * N1 * K + 255) / 256, cap = (int64_t)sm_count() * 32;
  edge_direct_kernel<T><<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(key, q, index, B, C, N2, N1, K,
                                                                                 include_query, out, status);
  return check_launch("edge_direct_kernel");
}

}  // namespace
}  // namespace tk3d

using namespace tk3d;

extern "C" size_t tk3d_edge_feature_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K,
                                                  int dtype) {
  if (dtype != TK3D_F32 || B <= 0 || B > 65535 || C < 4 || C > ROWS_MAX_C || C % 4 != 0 || N1 <= 0 || N2 <= 0 ||
      K <= 0 || (N1 * K) % 4 != 0 || N1 * K >= (1LL << 32) || (N2 + 31) / 32 > 65535)
    return 0;
  return rows_scratch_bytes(B, C, N2);
}

extern "C" int tk3d_edge_feature_fwd(const void *query_feature, const void *key_feature, const int64_t *index,
                                     int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K, int include_query,
                                     void *out, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                                     void *stream) {
  TK3D_RANGE("tk3d_edge_feature_fwd");
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "edge_feature_fwd: dtype %d", dtype);
  TK3D_REQUIRE(edge_shape_ok(B, C, N1, N2, K), TK3D_ERR_SHAPE, "edge_feature_fwd: bad size");
  if (B * C * N1 * K == 0) return TK3D_OK;
  TK3D_REQUIRE(query_feature && index && out && (key_feature || N2 == 0), TK3D_ERR_NULL,
               "edge_feature_fwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F64)
    return edge_fwd_direct<double>((const double *)key_feature, (const double *)query_feature, index, B, C, N2, N1, K,
                                   include_query, (double *)out, status, st);
  const size_t want = tk3d_edge_feature_scratch_bytes(B, C, N1, N2, K, dtype);
  const bool rows = want != 0 && scratch != nullptr && scratch_bytes >= want &&
                    ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scratch)) & 15) == 0;
  if (!rows)
    return edge_fwd_direct<float>((const float *)key_feature, (const float *)query_feature, index, B, C, N2, N1, K,
                                  include_query, (float *)out, status, st);
  int rc = transpose_bcn((const float *)key_feature, (float *)scratch, B, C, N2, st);
  if (rc) return rc;
  const size_t smem = (size_t)C * ROWS_TE * sizeof(float);
  if (smem > 48 * 1024)
    TK3D_CUDA(raise_smem_limit((const void *)edge_rows_vec4_kernel, (int)smem));
  dim3 grid((unsigned)((N1 * K + ROWS_TE - 1) / ROWS_TE), (unsigned)B);
  edge_rows_vec4_kernel<<<grid, ROWS_THREADS, smem, st>>>((const float *)scratch, (const float *)query_feature, index,
                                                          (int)C, N2, N1, (int)K, include_query, (float *)out,
                                                          status);
  return check_launch("edge_rows_vec4_kernel");
}

extern "C" int tk3d_edge_feature_bwd(const void *grad_out, const int64_t *index, int64_t B, int64_t C, int64_t N1,
                                     int64_t N2, int64_t K, int include_query, void *grad_query, void *grad_key,
                                     int32_t *status, void *scratch, size_t scratch_bytes, int dtype, void *stream) {
  TK3D_RANGE("tk3d_edge_feature_bwd");
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "edge_feature_bwd: dtype %d", dtype);
  TK3D_REQUIRE(edge_shape_ok(B, C, N1, N2, K), TK3D_ERR_SHAPE, "edge_feature_bwd: bad size");
  const int64_t E = N1 * K;
  TK3D_REQUIRE(B * C * E == 0 || (grad_out && index), TK3D_ERR_NULL, "edge_feature_bwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t gstride = (include_query ? 2 * C : C) * E;
  const size_t elem = dtype == TK3D_F64 ? 8 : 4;
  if (grad_query && B * C * N1 > 0) {
    const int64_t blocks = (B * C * N1 + 255) / 256, cap = (int64_t)sm_count() * 32;
    const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
    if (dtype == TK3D_F32)
      edge_bwd_query_kernel<float><<<grid, 256, 0, st>>>((const float *)grad_out, B, C, N1, K, include_query,
                                                         (float *)grad_query);
    else
      edge_bwd_query_kernel<double><<<grid, 256, 0, st>>>((const double *)grad_out, B, C, N1, K, include_query,
                                                          (double *)grad_query);
    int rc = check_launch("edge_bwd_query_kernel");
    if (rc) return rc;
  }
  if (grad_key && B * C * N2 > 0) {
    const size_t want = tk3d_edge_feature_scratch_bytes(B, C, N1, N2, K, dtype);
    const bool rows = want != 0 && scratch != nullptr && scratch_bytes >= want && rows_vec_ok(C, E, grad_out, scratch);
    if (rows) {
      TK3D_CUDA(cudaMemsetAsync(scratch, 0, want, st));
      const size_t smem = (size_t)C * ROWS_TE * sizeof(float);
      if (smem > 48 * 1024)
        TK3D_CUDA(raise_smem_limit((const void *)scatter_rows_vec4_kernel<1, int64_t>, (int)smem));
      dim3 grid((unsigned)((E + ROWS_TE - 1) / ROWS_TE), (unsigned)B);
      scatter_rows_vec4_kernel<1, int64_t><<<grid, ROWS_THREADS, smem, st>>>(
          (const float *)grad_out, index, nullptr, (int)C, N2, E, gstride, (float *)scratch, status);
      int rc = check_launch("scatter_rows_vec4_kernel");
      if (rc) return rc;
      return transpose_bcn((const float *)scratch, (float *)grad_key, B, N2, C, st);
    }
    TK3D_CUDA(cudaMemsetAsync(grad_key, 0, elem * (size_t)(B * C * N2), st));
    if (E > 0) {
      const int64_t blocks = (B * C * E + 255) / 256, cap = (int64_t)sm_count() * 32;
      const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
      if (dtype == TK3D_F32)
        edge_bwd_key_kernel<float><<<grid, 256, 0, st>>>((const float *)grad_out, index, B, C, N2, E, gstride,
                                                         (float *)grad_key, status);
      else
        edge_bwd_key_kernel<double><<<grid, 256, 0, st>>>((const double *)grad_out, index, B, C, N2, E, gstride,
                                                          (double *)grad_key, status);
      int rc = check_launch("edge_bwd_key_kernel");
      if (rc) return rc;
    }
  }
  return TK3D_OK;
}

TK3D_BOUNDS_TU(edge)
