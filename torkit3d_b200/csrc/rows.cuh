// Row gathers for the memory-bound operators (group_points and interpolation, fp32).
//
// Gathering from the native [B,C,N1] feature layout touches one 4-byte element per 32-byte sector
// for every (channel, index) pair, so most of the L2->SM traffic is wasted.  When the output is
// much larger than the feature tensor it pays to transpose the features once into a caller
// provided scratch [B,N1,C]: every gathered row is then C contiguous floats (fully used sectors,
// coalesced 128-byte warp loads), and the block turns the rows back into the channel-major output
// through a shared-memory tile so that global stores stay coalesced along the entry axis.
#pragma once

#include "tk3d_common.cuh"

namespace tk3d {

constexpr int ROWS_TE = 64;        // entries (index positions) per block
constexpr int ROWS_THREADS = 256;  // 8 warps
constexpr int ROWS_MAX_C = 512;

// in [B][C][N] -> out [B][N][C]
static __global__ void __launch_bounds__(256) transpose_bcn_kernel(const float *__restrict__ in, float *__restrict__ out,
                                                            int C, int64_t N) {
  __shared__ float t[32][33];
  const int64_t b = blockIdx.z;
  const int64_t n0 = (int64_t)blockIdx.x * 32;
  const int c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const float *src = in + b * C * N;
  float *dst = out + b * N * C;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty + 8 * i;
    const int64_t n = n0 + tx;
    if (c < C && n < N) t[ty + 8 * i][tx] = src[(int64_t)c * N + n];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t n = n0 + ty + 8 * i;
    const int c = c0 + tx;
    if (c < C && n < N) dst[n * C + c] = t[tx][ty + 8 * i];
  }
}

// NSRC = 1: out[b,c,e] = featT[b, index[b,e], c]                       (group_points, e = m*K + j)
// NSRC = 3: out[b,c,e] = sum_i featT[b, index[b,e,i], c] * weight[b,e,i]  (interpolation, e = m)
// An index outside [0,N1) contributes 0 and raises bit 0 of *status.
template <int NSRC, typename IndexT = int64_t>
__global__ void __launch_bounds__(ROWS_THREADS)
gather_rows_kernel(const float *__restrict__ featT, const IndexT *__restrict__ index,
                   const float *__restrict__ weight, int C, int64_t N1, int64_t E, float *__restrict__ out,
                   int32_t *__restrict__ status) {
  extern __shared__ float tile[];  // [C][ROWS_TE + 1]
  __shared__ int sidx[ROWS_TE * NSRC];
  __shared__ float sw[ROWS_TE * NSRC];
  constexpr int S = ROWS_TE + 1;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t b = blockIdx.y;
  const int64_t e0 = (int64_t)blockIdx.x * ROWS_TE;
  const int n = (int)((E - e0) < ROWS_TE ? (E - e0) : ROWS_TE);

  bool bad = false;
  for (int t = tid; t < n * NSRC; t += ROWS_THREADS) {
    int64_t id = index[(b * E + e0) * NSRC + t];
    if (id < 0 || id >= N1) {
      id = -1;
      bad = true;
    }
    sidx[t] = (int)id;
    if (NSRC == 3) sw[t] = weight[(b * E + e0) * NSRC + t];
  }
  if (bad && status) atomicOr(status, 1);
  __syncthreads();

  const float *fb = featT + b * N1 * C;
  for (int e = warp; e < n; e += ROWS_THREADS / 32) {
    if (NSRC == 1) {
      const int id = sidx[e];
      const float *row = fb + (int64_t)(id < 0 ? 0 : id) * C;
      for (int c = lane; c < C; c += 32) tile[c * S + e] = id < 0 ? 0.f : __ldg(row + c);
    } else {
      const int i0 = sidx[3 * e], i1 = sidx[3 * e + 1], i2 = sidx[3 * e + 2];
      const float w0 = i0 < 0 ? 0.f : sw[3 * e], w1 = i1 < 0 ? 0.f : sw[3 * e + 1], w2 = i2 < 0 ? 0.f : sw[3 * e + 2];
      const float *r0 = fb + (int64_t)(i0 < 0 ? 0 : i0) * C;
      const float *r1 = fb + (int64_t)(i1 < 0 ? 0 : i1) * C;
      const float *r2 = fb + (int64_t)(i2 < 0 ? 0 : i2) * C;
      for (int c = lane; c < C; c += 32) {
        float acc = __ldg(r0 + c) * w0;
        acc += __ldg(r1 + c) * w1;
        acc += __ldg(r2 + c) * w2;
        tile[c * S + e] = acc;
      }
    }
  }
  __syncthreads();

  float *ob = out + b * C * E + e0;
  for (int c = warp; c < C; c += ROWS_THREADS / 32) {
    for (int e = lane; e < n; e += 32) __stcs(ob + (int64_t)c * E + e, tile[c * S + e]);
  }
}

// Vectorised variant for C % 4 == 0, E % 4 == 0 and 16-byte aligned buffers: 16-byte global loads
// (consecutive lanes read consecutive float4 of one row), a [C][64] tile whose 16-byte chunks are
// XOR-swizzled by the channel group so that the transposing scalar stores are at most 4-way
// conflicted and the float4 reads of the second phase are conflict-free, and 16-byte streaming
// stores of four consecutive entries per lane.
template <int NSRC, typename IndexT = int64_t>
__global__ void __launch_bounds__(ROWS_THREADS)
gather_rows_vec4_kernel(const float *__restrict__ featT, const IndexT *__restrict__ index,
                        const float *__restrict__ weight, int C, int64_t N1, int64_t E, float *__restrict__ out,
                        int32_t *__restrict__ status) {
  extern __shared__ __align__(16) float tile[];  // [C][ROWS_TE], chunk-swizzled
  __shared__ int sidx[ROWS_TE * NSRC];
  __shared__ float sw[ROWS_TE * NSRC];
  const int tid = threadIdx.x;
  const int64_t b = blockIdx.y;
  const int64_t e0 = (int64_t)blockIdx.x * ROWS_TE;
  const int n = (int)((E - e0) < ROWS_TE ? (E - e0) : ROWS_TE);  // multiple of 4
  const int L = C >> 2;                                           // float4 per row

  bool bad = false;
  for (int t = tid; t < n * NSRC; t += ROWS_THREADS) {
    int64_t id = index[(b * E + e0) * NSRC + t];
    if (id < 0 || id >= N1) {
      id = -1;
      bad = true;
    }
    sidx[t] = (int)id;
    if (NSRC == 3) sw[t] = weight[(b * E + e0) * NSRC + t];
  }
  if (bad && status) atomicOr(status, 1);
  __syncthreads();

  // Phase 1: item t = e * L + q  (entry e, float4 q of its row); consecutive threads take
  // consecutive items, so a warp reads whole contiguous row pieces.
  const float4 *fb = reinterpret_cast<const float4 *>(featT + b * N1 * C);
  const int items = n * L;
  int e = tid / L, q = tid - e * L;
  const int de = ROWS_THREADS / L, dq = ROWS_THREADS - de * L;
  for (int t = tid; t < items; t += ROWS_THREADS) {
    float4 v;
    if (NSRC == 1) {
      const int id = sidx[e];
      v = id < 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : __ldg(fb + (int64_t)id * L + q);
    } else {
      const int i0 = sidx[3 * e], i1 = sidx[3 * e + 1], i2 = sidx[3 * e + 2];
      const float w0 = i0 < 0 ? 0.f : sw[3 * e], w1 = i1 < 0 ? 0.f : sw[3 * e + 1], w2 = i2 < 0 ? 0.f : sw[3 * e + 2];
      const float4 f0 = __ldg(fb + (int64_t)(i0 < 0 ? 0 : i0) * L + q);
      const float4 f1 = __ldg(fb + (int64_t)(i1 < 0 ? 0 : i1) * L + q);
      const float4 f2 = __ldg(fb + (int64_t)(i2 < 0 ? 0 : i2) * L + q);
      v.x = f0.x * w0;
      v.y = f0.y * w0;
      v.z = f0.z * w0;
      v.w = f0.w * w0;
      v.x += f1.x * w1;
      v.y += f1.y * w1;
      v.z += f1.z * w1;
      v.w += f1.w * w1;
      v.x += f2.x * w2;
      v.y += f2.y * w2;
      v.z += f2.z * w2;
      v.w += f2.w * w2;
    }
    // channel c = 4q + i lives in row c; entry e sits in chunk ((e >> 2) ^ q) & 15, slot e & 3
    float *dst = tile + (4 * q) * ROWS_TE + ((((e >> 2) ^ q) & (ROWS_TE / 4 - 1)) << 2) + (e & 3);
    dst[0] = v.x;
    dst[ROWS_TE] = v.y;
    dst[2 * ROWS_TE] = v.z;
    dst[3 * ROWS_TE] = v.w;
    e += de;
    q += dq;
    if (q >= L) {
      q -= L;
      ++e;
    }
  }
  __syncthreads();

  // Phase 2: item u = c * 16 + chunk; a lane moves four consecutive entries of one channel.
  const int nchunks = n >> 2;
  float *ob = out + b * C * E + e0;
  for (int u = tid; u < C * (ROWS_TE / 4); u += ROWS_THREADS) {
    const int c = u >> 4, ch = u & 15;
    if (ch < nchunks) {
      const float4 v = *reinterpret_cast<const float4 *>(tile + c * ROWS_TE + (((ch ^ (c >> 2)) & 15) << 2));
      __stcs(reinterpret_cast<float4 *>(ob + (int64_t)c * E + 4 * ch), v);
    }
  }
}

// 16-byte vector reduction: four consecutive floats of one row in a single L2 atomic operation.
__device__ __forceinline__ void red_add4(float *p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Backward of the row gathers: gradT[b, index[b,e(,i)], :] += gout[b, :, e] (* weight[b,e,i]) into a
// zeroed transposed accumulator [B,N1,C], which the host transposes back afterwards.  The tile of
// gout is read with 16-byte loads along the entry axis, turned into rows through the same swizzled
// shared-memory tile as the forward, and every lane issues 16-byte vector reductions on contiguous
// row pieces, so the L2 atomics work on full sectors instead of scattered single floats.
// `gstride` is the distance in elements between the gout slabs of consecutive clouds (C*E when gout
// is a dense [B,C,E] tensor; larger when the C channels are the leading part of a wider tensor).
template <int NSRC, typename IndexT = int64_t>
__global__ void __launch_bounds__(ROWS_THREADS)
scatter_rows_vec4_kernel(const float *__restrict__ gout, const IndexT *__restrict__ index,
                         const float *__restrict__ weight, int C, int64_t N1, int64_t E, int64_t gstride,
                         float *__restrict__ gradT, int32_t *__restrict__ status) {
  extern __shared__ __align__(16) float tile[];  // [C][ROWS_TE], chunk-swizzled
  __shared__ int sidx[ROWS_TE * NSRC];
  __shared__ float sw[ROWS_TE * NSRC];
  const int tid = threadIdx.x;
  const int64_t b = blockIdx.y;
  const int64_t e0 = (int64_t)blockIdx.x * ROWS_TE;
  const int n = (int)((E - e0) < ROWS_TE ? (E - e0) : ROWS_TE);  // multiple of 4
  const int L = C >> 2;

  bool bad = false;
  for (int t = tid; t < n * NSRC; t += ROWS_THREADS) {
    int64_t id = index[(b * E + e0) * NSRC + t];
    if (id < 0 || id >= N1) {
      id = -1;
      bad = true;
    }
    sidx[t] = (int)id;
    if (NSRC == 3) sw[t] = weight[(b * E + e0) * NSRC + t];
  }
  if (bad && status) atomicOr(status, 1);

  // Phase 1: gout[b, c, e0 + 4*ch ..] -> tile row c, swizzled chunk.
  const int nchunks = n >> 2;
  const float *gb = gout + b * gstride + e0;
  for (int u = tid; u < C * (ROWS_TE / 4); u += ROWS_THREADS) {
    const int c = u >> 4, ch = u & 15;
    if (ch < nchunks) {
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(gb + (int64_t)c * E + 4 * ch));
      *reinterpret_cast<float4 *>(tile + c * ROWS_TE + (((ch ^ (c >> 2)) & 15) << 2)) = v;
    }
  }
  __syncthreads();

  // Phase 2: item t = e * L + q -> four channels of entry e, reduced into the row(s) of its index.
  float *tb = gradT + b * N1 * C;
  const int items = n * L;
  int e = tid / L, q = tid - e * L;
  const int de = ROWS_THREADS / L, dq = ROWS_THREADS - de * L;
  for (int t = tid; t < items; t += ROWS_THREADS) {
    const float *src = tile + (4 * q) * ROWS_TE + ((((e >> 2) ^ q) & (ROWS_TE / 4 - 1)) << 2) + (e & 3);
    const float vx = src[0], vy = src[ROWS_TE], vz = src[2 * ROWS_TE], vw = src[3 * ROWS_TE];
    if (NSRC == 1) {
      const int id = sidx[e];
      if (id >= 0) red_add4(tb + (int64_t)id * C + 4 * q, vx, vy, vz, vw);
    } else {
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        const int id = sidx[3 * e + i];
        const float w = sw[3 * e + i];
        if (id >= 0) red_add4(tb + (int64_t)id * C + 4 * q, vx * w, vy * w, vz * w, vw * w);
      }
    }
    e += de;
    q += dq;
    if (q >= L) {
      q -= L;
      ++e;
    }
  }
}

inline size_t rows_scratch_bytes(int64_t B, int64_t C, int64_t N1) { return (size_t)B * (size_t)C * (size_t)N1 * 4; }

// Worth it when the gathered output is at least twice the feature tensor and C fits a tile.
inline bool rows_profitable(int64_t C, int64_t N1, int64_t E, int nsrc) {
  return C >= 16 && C <= ROWS_MAX_C && N1 > 0 && E * nsrc >= 2 * N1;
}

template <int NSRC, typename IndexT = int64_t>
int gather_rows(const float *in, const IndexT *index, const float *weight, int64_t B, int64_t C, int64_t N1,
                int64_t E, float *out, int32_t *status, float *scratch, cudaStream_t st) {
  TK3D_REQUIRE(B <= 65535, TK3D_ERR_SHAPE, "gather: batch too large for this path (B=%lld)", (long long)B);
  dim3 tg((unsigned)((N1 + 31) / 32), (unsigned)((C + 31) / 32), (unsigned)B);
  transpose_bcn_kernel<<<tg, 256, 0, st>>>(in, scratch, (int)C, N1);
  int rc = check_launch("transpose_bcn_kernel");
  if (rc) return rc;
  dim3 grid((unsigned)((E + ROWS_TE - 1) / ROWS_TE), (unsigned)B);
  const bool vec = C % 4 == 0 && E % 4 == 0 && ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scratch)) & 15) == 0;
  if (vec) {
    const size_t smem = (size_t)C * ROWS_TE * sizeof(float);
    if (smem > 48 * 1024)
      TK3D_CUDA(raise_smem_limit((const void *)gather_rows_vec4_kernel<NSRC, IndexT>, (int)smem));
    gather_rows_vec4_kernel<NSRC, IndexT><<<grid, ROWS_THREADS, smem, st>>>(scratch, index, weight, (int)C, N1, E, out,
                                                                    status);
    return check_launch("gather_rows_vec4_kernel");
  }
  const size_t smem = (size_t)C * (ROWS_TE + 1) * sizeof(float);
  if (smem > 48 * 1024)
    TK3D_CUDA(raise_smem_limit((const void *)gather_rows_kernel<NSRC, IndexT>, (int)smem));
  gather_rows_kernel<NSRC, IndexT><<<grid, ROWS_THREADS, smem, st>>>(scratch, index, weight, (int)C, N1, E, out, status);
  return check_launch("gather_rows_kernel");
}

// Backward through the transposed accumulator; `vec_ok` has been checked by the caller.
template <int NSRC>
int scatter_rows(const float *gout, const int64_t *index, const float *weight, int64_t B, int64_t C, int64_t N1,
                 int64_t E, float *gin, int32_t *status, float *scratch, cudaStream_t st) {
  TK3D_REQUIRE(B <= 65535 && (N1 + 31) / 32 <= 65535, TK3D_ERR_SHAPE, "scatter: size too large for this path");
  TK3D_CUDA(cudaMemsetAsync(scratch, 0, rows_scratch_bytes(B, C, N1), st));
  if (E > 0) {
    const size_t smem = (size_t)C * ROWS_TE * sizeof(float);
    if (smem > 48 * 1024)
      TK3D_CUDA(raise_smem_limit((const void *)scatter_rows_vec4_kernel<NSRC>, (int)smem));
    dim3 grid((unsigned)((E + ROWS_TE - 1) / ROWS_TE), (unsigned)B);
    scatter_rows_vec4_kernel<NSRC><<<grid, ROWS_THREADS, smem, st>>>(gout, index, weight, (int)C, N1, E, C * E,
                                                                     scratch, status);
    int rc = check_launch("scatter_rows_vec4_kernel");
    if (rc) return rc;
  }
  // scratch [B][N1][C] -> gin [B][C][N1]: the same tile transpose with the roles of the axes swapped
  dim3 tg((unsigned)((C + 31) / 32), (unsigned)((N1 + 31) / 32), (unsigned)B);
  transpose_bcn_kernel<<<tg, 256, 0, st>>>(scratch, gin, (int)N1, C);
  return check_launch("transpose_bcn_kernel");
}

inline bool rows_vec_ok(int64_t C, int64_t E, const void *a, const void *b) {
  return C % 4 == 0 && E % 4 == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
}

}  // namespace tk3d
