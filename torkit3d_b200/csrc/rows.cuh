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

constexpr int ROWS_TE = 32;        // entries (index positions) per block
constexpr int ROWS_THREADS = 128;  // 4 warps
constexpr int ROWS_MAX_C = 512;
constexpr int ROWS_CH = ROWS_TE / 4;   // 16-byte chunks (four entries) per tile row
constexpr int ROWS_GPW = ROWS_TE / 4 / (ROWS_THREADS / 32);  // entry groups (of four) per warp

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

// The same transposition with 16-byte accesses on both sides, for C % 4 == 0, N % 4 == 0 and
// 16-byte aligned buffers: a block moves a 64 x 64 tile.  Loading, a warp covers four channel rows
// at a time (lane = 8 * el + ql reads float4 number ql or ql + 8 of row 4g + el) and stores the four
// values as scalars into a [n][64 c] tile whose 16-byte chunk of channels 4g .. 4g+3 sits at chunk
// position (g ^ (n >> 2)) & 15: the 32 stores of one instruction fall into 32 different banks.
// Storing, a lane moves four consecutive channels of one n with a conflict-free 16-byte shared load.
static __global__ void __launch_bounds__(256) transpose_bcn_vec4_kernel(const float *__restrict__ in,
                                                                        float *__restrict__ out, int C, int64_t N) {
  __shared__ __align__(16) float t[64 * 64];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ql = lane & 7, el = lane >> 3;
  const int64_t b = blockIdx.z;
  const int64_t n0 = (int64_t)blockIdx.x * 64;
  const int c0 = blockIdx.y * 64;
  const float *src = in + b * C * N;
  float *dst = out + b * N * C;
#pragma unroll
  for (int g = warp; g < 16; g += 8) {
    const int c = c0 + 4 * g + el;
#pragma unroll
    for (int q = ql; q < 16; q += 8) {
      const int64_t n = n0 + 4 * q;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < C && n < N) v = __ldg(reinterpret_cast<const float4 *>(src + (int64_t)c * N + n));
      float *p = t + (4 * q) * 64 + (((g ^ q) & 15) << 2) + el;
      p[0] = v.x;
      p[64] = v.y;
      p[128] = v.z;
      p[192] = v.w;
    }
  }
  __syncthreads();
#pragma unroll
  for (int u = tid; u < 64 * 16; u += 256) {
    const int nl = u >> 4, ch = u & 15;
    const int64_t n = n0 + nl;
    const int c = c0 + 4 * ch;
    if (n < N && c < C) {
      const float4 v = *reinterpret_cast<const float4 *>(t + nl * 64 + (((ch ^ (nl >> 2)) & 15) << 2));
      *reinterpret_cast<float4 *>(dst + n * C + c) = v;
    }
  }
}

// in [B][C][N] -> out [B][N][C] on stream st; picks the 16-byte kernel when sizes and alignment allow.
inline int transpose_bcn(const float *in, float *out, int64_t B, int64_t C, int64_t N, cudaStream_t st) {
  if (B <= 0 || C <= 0 || N <= 0) return TK3D_OK;
  TK3D_REQUIRE(B <= 65535, TK3D_ERR_SHAPE, "transpose: batch too large for this path (B=%lld)", (long long)B);
  const bool vec = C % 4 == 0 && N % 4 == 0 && C >= 16 && N >= 16 &&
                   ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (vec && (C + 63) / 64 <= 65535) {
    dim3 tg((unsigned)((N + 63) / 64), (unsigned)((C + 63) / 64), (unsigned)B);
    transpose_bcn_vec4_kernel<<<tg, 256, 0, st>>>(in, out, (int)C, N);
    return check_launch("transpose_bcn_vec4_kernel");
  }
  TK3D_REQUIRE((C + 31) / 32 <= 65535, TK3D_ERR_SHAPE, "transpose: size too large for this path");
  dim3 tg((unsigned)((N + 31) / 32), (unsigned)((C + 31) / 32), (unsigned)B);
  transpose_bcn_kernel<<<tg, 256, 0, st>>>(in, out, (int)C, N);
  return check_launch("transpose_bcn_kernel");
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

// Vectorised variant for C % 4 == 0, E % 4 == 0 and 16-byte aligned buffers.  The tile is
// [C][ROWS_TE] floats; the 16-byte chunk holding entries 4g .. 4g+3 of channel c sits at chunk
// position (g ^ (c >> 2)) & (ROWS_TE / 4 - 1) of row c.  Tiles are small (32 entries, four warps):
// a barrier then holds few warps and ten blocks fit an SM, which measured 10 % faster than 64
// entries with eight warps on the interpolation gather.
//
// Phase 1 -- a warp works on four entries at a time: lane = 8 * el + ql reads, for entry 4g + el,
// the float4 number 8 * qh + ql of its row(s) (eight consecutive lanes cover 128 contiguous
// bytes) and stores its four channels as scalars.  For one store instruction the bank is
// 4 * ((g ^ ql) & 7) + el: all 32 lanes hit different banks.  (With one entry per warp, the
// previous mapping, the 32 stores could only reach the 8 banks congruent to e & 3 -- four
// wavefronts per store, and the kernel was bound by the shared-memory data path.)  Indices and
// weights are read straight from global memory, once per group of four entries.
// Phase 2 -- a lane moves four consecutive entries of one channel: conflict-free 16-byte shared
// loads, 16-byte streaming stores.
template <int NSRC, typename IndexT>
__device__ __forceinline__ void rows_load_index(const IndexT *__restrict__ index, const float *__restrict__ weight,
                                                int64_t at, int64_t N1, bool live, int (&id)[NSRC], float (&w)[NSRC],
                                                bool &bad) {
#pragma unroll
  for (int i = 0; i < NSRC; ++i) {
    int64_t v = live ? (int64_t)index[at * NSRC + i] : 0;  // a group beyond the tile reads nothing
    w[i] = 1.f;
    if (NSRC > 1) w[i] = live ? weight[at * NSRC + i] : 0.f;
    if (v < 0 || v >= N1) {
      v = -1;
      bad = true;
    }
    id[i] = (int)v;
  }
}

template <int NSRC, typename IndexT = int64_t>
__global__ void __launch_bounds__(ROWS_THREADS, 10)
gather_rows_vec4_kernel(const float *__restrict__ featT, const IndexT *__restrict__ index,
                        const float *__restrict__ weight, int C, int64_t N1, int64_t E, float *__restrict__ out,
                        int32_t *__restrict__ status) {
  extern __shared__ __align__(16) float tile[];  // [C][ROWS_TE], chunk-swizzled
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ql = lane & 7, el = lane >> 3;
  const int64_t b = blockIdx.y;
  const int64_t e0 = (int64_t)blockIdx.x * ROWS_TE;
  const int n = (int)((E - e0) < ROWS_TE ? (E - e0) : ROWS_TE);  // multiple of 4
  const int L = C >> 2;                                           // float4 per row

  const float4 *fb = reinterpret_cast<const float4 *>(featT + b * N1 * C);
  bool bad = false;
  // a warp owns the entry groups warp and warp + 4; the indices and weights of both are requested
  // before the first row load, so the second group does not pay that latency again
  int ids[ROWS_GPW][NSRC];
  float ws[ROWS_GPW][NSRC];
#pragma unroll
  for (int j = 0; j < ROWS_GPW; ++j) {
    const int g = warp + j * (ROWS_THREADS / 32);
    rows_load_index<NSRC, IndexT>(index, weight, b * E + e0 + 4 * g + el, N1, g < (n >> 2), ids[j], ws[j], bad);
  }
#pragma unroll
  for (int j = 0; j < ROWS_GPW; ++j) {
    const int g = warp + j * (ROWS_THREADS / 32);
    if (g >= (n >> 2)) break;
    int (&id)[NSRC] = ids[j];
    float (&w)[NSRC] = ws[j];
    const float4 *row[NSRC];
#pragma unroll
    for (int i = 0; i < NSRC; ++i) {
      row[i] = fb + (int64_t)(id[i] < 0 ? 0 : id[i]) * L;
      if (id[i] < 0) w[i] = 0.f;
    }
#pragma unroll 2
    for (int q = ql; q < L; q += 8) {
      float4 v;
      if (NSRC == 1) {
        v = id[0] < 0 ? make_float4(0.f, 0.f, 0.f, 0.f) : __ldg(row[0] + q);
      } else {
        const float4 f0 = __ldg(row[0] + q);
        const float4 f1 = __ldg(row[NSRC > 1 ? 1 : 0] + q);
        const float4 f2 = __ldg(row[NSRC > 2 ? 2 : 0] + q);
        v.x = f0.x * w[0];
        v.y = f0.y * w[0];
        v.z = f0.z * w[0];
        v.w = f0.w * w[0];
        v.x += f1.x * w[NSRC > 1 ? 1 : 0];
        v.y += f1.y * w[NSRC > 1 ? 1 : 0];
        v.z += f1.z * w[NSRC > 1 ? 1 : 0];
        v.w += f1.w * w[NSRC > 1 ? 1 : 0];
        v.x += f2.x * w[NSRC > 2 ? 2 : 0];
        v.y += f2.y * w[NSRC > 2 ? 2 : 0];
        v.z += f2.z * w[NSRC > 2 ? 2 : 0];
        v.w += f2.w * w[NSRC > 2 ? 2 : 0];
      }
      float *dst = tile + (4 * q) * ROWS_TE + (((g ^ q) & (ROWS_TE / 4 - 1)) << 2) + el;
      dst[0] = v.x;
      dst[ROWS_TE] = v.y;
      dst[2 * ROWS_TE] = v.z;
      dst[3 * ROWS_TE] = v.w;
    }
  }
  if (bad && status) atomicOr(status, 1);
  __syncthreads();

  // Phase 2: item u = c * 16 + chunk; a lane moves four consecutive entries of one channel.
  const int nchunks = n >> 2;
  float *ob = out + b * C * E + e0;
  for (int u = tid; u < C * (ROWS_TE / 4); u += ROWS_THREADS) {
    const int c = u / ROWS_CH, ch = u % ROWS_CH;
    if (ch < nchunks) {
      const float4 v = *reinterpret_cast<const float4 *>(tile + c * ROWS_TE + (((ch ^ (c >> 2)) & (ROWS_CH - 1)) << 2));
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
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ql = lane & 7, el = lane >> 3;
  const int64_t b = blockIdx.y;
  const int64_t e0 = (int64_t)blockIdx.x * ROWS_TE;
  const int n = (int)((E - e0) < ROWS_TE ? (E - e0) : ROWS_TE);  // multiple of 4
  const int L = C >> 2;

  // Phase 1: gout[b, c, e0 + 4*ch ..] -> tile row c, swizzled chunk.
  const int nchunks = n >> 2;
  const float *gb = gout + b * gstride + e0;
  for (int u = tid; u < C * (ROWS_TE / 4); u += ROWS_THREADS) {
    const int c = u / ROWS_CH, ch = u % ROWS_CH;
    if (ch < nchunks) {
      const float4 v = __ldcs(reinterpret_cast<const float4 *>(gb + (int64_t)c * E + 4 * ch));
      *reinterpret_cast<float4 *>(tile + c * ROWS_TE + (((ch ^ (c >> 2)) & (ROWS_CH - 1)) << 2)) = v;
    }
  }
  // indices and weights of this warp's two entry groups, requested before the barrier
  bool bad = false;
  int ids[ROWS_GPW][NSRC];
  float ws[ROWS_GPW][NSRC];
#pragma unroll
  for (int j = 0; j < ROWS_GPW; ++j) {
    const int g = warp + j * (ROWS_THREADS / 32);
    rows_load_index<NSRC, IndexT>(index, weight, b * E + e0 + 4 * g + el, N1, g < nchunks, ids[j], ws[j], bad);
  }
  __syncthreads();

  // Phase 2: the lane mapping of the forward kernel's phase 1 (four entries per warp, conflict-free
  // scalar reads): four channels of entry 4g + el, reduced into the row(s) of its index.
  float *tb = gradT + b * N1 * C;
#pragma unroll
  for (int j = 0; j < ROWS_GPW; ++j) {
    const int g = warp + j * (ROWS_THREADS / 32);
    if (g >= nchunks) break;
    int (&id)[NSRC] = ids[j];
    float (&w)[NSRC] = ws[j];
#pragma unroll 4
    for (int q = ql; q < L; q += 8) {
      const float *src = tile + (4 * q) * ROWS_TE + (((g ^ q) & (ROWS_TE / 4 - 1)) << 2) + el;
      const float vx = src[0], vy = src[ROWS_TE], vz = src[2 * ROWS_TE], vw = src[3 * ROWS_TE];
#pragma unroll
      for (int i = 0; i < NSRC; ++i) {
        if (id[i] >= 0) red_add4(tb + (int64_t)id[i] * C + 4 * q, vx * w[i], vy * w[i], vz * w[i], vw * w[i]);
      }
    }
  }
  if (bad && status) atomicOr(status, 1);
}

inline size_t rows_scratch_bytes(int64_t B, int64_t C, int64_t N1) { return (size_t)B * (size_t)C * (size_t)N1 * 4; }

// Worth it when the output is at least a quarter of the feature tensor and C fits a tile: the
// transposition moves the features at the HBM copy rate, the row gather then costs about a seventh
// of the direct gather per output byte (measured on B200: 0.35 us per MB of features + 0.37 us per
// MB of output against 2.7 us per MB of output).
inline bool rows_profitable(int64_t C, int64_t N1, int64_t E, int nsrc) {
  (void)nsrc;
  return C >= 16 && C <= ROWS_MAX_C && N1 > 0 && 4 * E >= N1;
}

// The gather alone, from features that already lie as rows [B,N1,C].
template <int NSRC, typename IndexT = int64_t>
int gather_from_rows(const float *scratch, const IndexT *index, const float *weight, int64_t B, int64_t C, int64_t N1,
                     int64_t E, float *out, int32_t *status, cudaStream_t st) {
  TK3D_REQUIRE(B <= 65535, TK3D_ERR_SHAPE, "gather: batch too large for this path (B=%lld)", (long long)B);
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

// Transposition into caller scratch, then the gather.
template <int NSRC, typename IndexT = int64_t>
int gather_rows(const float *in, const IndexT *index, const float *weight, int64_t B, int64_t C, int64_t N1,
                int64_t E, float *out, int32_t *status, float *scratch, cudaStream_t st) {
  int rc = transpose_bcn(in, scratch, B, C, N1, st);
  if (rc) return rc;
  return gather_from_rows<NSRC, IndexT>(scratch, index, weight, B, C, N1, E, out, status, st);
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
  return transpose_bcn(scratch, gin, B, N1, C, st);
}

inline bool rows_vec_ok(int64_t C, int64_t E, const void *a, const void *b) {
  return C % 4 == 0 && E % 4 == 0 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
}

}  // namespace tk3d
