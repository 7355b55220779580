// Fused front end of a PointNet++ set-abstraction layer (fp32):
//     index   = ball_query(centroids, points, radius, K)
//     out     = cat([group_points(feature, index), group_points(points, index) - centroids[..., None]], dim=1)
// in one kernel.  The neighbour lists never leave shared memory as 64-bit indices and the grouped,
// un-centred coordinates are never materialised; the concatenated [B, C+3, M, K] tensor that feeds
// the shared MLP is written once, directly.  A 32-bit copy of the index is written only on request
// (the backward needs it).
//
// A block of 4 warps owns 32 centroids of one cloud.
//   Phase A (compute bound): lane = centroid; warp s sweeps the s-th quarter of every 256-point
//     tile with the filter-then-verify test of sweep.cuh and keeps an ascending hit list per
//     (quarter, centroid); the four lists are merged by point index, which reproduces "first K in
//     index order, padded with the first hit, -1 when there is none" bit for bit.
//   Phase B (memory bound): the 32*K rows named by the merged lists are fetched from the
//     channel-last copy of the features with 16-byte loads, turned into channel-major order
//     through a chunk-swizzled shared tile (which reuses the memory of phase A) and stored with
//     16-byte streaming stores; the three coordinate channels are gathered, centred and stored by
//     the same block.
// Measured on B200 (B=32, 8192 points, 1024 centres, K=32, C=64): 0.25 ms against 0.37 ms for the
// same result spelled as ball query + two gathers + subtraction + concatenation.  With this shape
// all 1024 blocks are resident at once and pass through the two phases together, so the time is
// close to the sum of a ball query (0.13 ms) and a gather (0.11 ms); larger batches, whose blocks
// come in several waves, let the sweep of one block overlap the traffic of another.
#include "rows.cuh"
#include "sweep.cuh"

namespace tk3d {

namespace {

constexpr int SA_TILE = 256;   // points per staged tile
constexpr int SA_Q = 32;       // centroids per block
constexpr int SA_MAX_K = 128;
constexpr int SA_TE = 64;      // entries per gather sub-tile

struct SaSmem {
  size_t sidx, gtile, total;
};

// Dynamic shared memory: [sidx | union(phase A: key tiles, phase B: gather tile)].
inline SaSmem sa_smem(int C, int K, bool vec) {
  SaSmem s;
  s.sidx = sizeof(int) * SA_Q * (size_t)(K + 1);
  s.sidx = (s.sidx + 15) & ~(size_t)15;
  const size_t phase_a = sizeof(float4) * 2 * SA_TILE;
  s.gtile = sizeof(float) * (size_t)C * (vec ? SA_TE : SA_TE + 1);
  s.total = s.sidx + (phase_a > s.gtile ? phase_a : s.gtile);
  return s;
}

// Point j, coordinate d of cloud b lives at base[b*3*N + j*ps + d*cs]: (ps, cs) = (3, 1) for
// [B,N,3] and (1, N) for [B,3,N].
template <int SPLIT>
__global__ void __launch_bounds__(32 * SPLIT)
sa_group_fwd_kernel(const float *__restrict__ points, const float *__restrict__ centroids,
                    const float *__restrict__ featT, int64_t B, int C, int N, int M, int pps, int pcs, int cps,
                    int cpc, float r2, int K, int use_xyz, int vec, float *__restrict__ out,
                    int32_t *__restrict__ index32, int32_t *__restrict__ status, int64_t blocks_total) {
  constexpr int THREADS = 32 * SPLIT;  // SPLIT warps share every tile of points
  constexpr int PER = SA_TILE / THREADS;
  constexpr int QK = SA_TILE / SPLIT;
  static_assert(PER >= 1, "a tile is staged by one pass of the block");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  static_assert(QK <= 64, "a slice's hits are kept as a 64-bit mask");
  __shared__ int tcount[2][SPLIT][SA_Q];
  __shared__ float scent[3][SA_Q];
  const int S1 = K + 1;  // padded row length of the hit lists
  int *sidx = reinterpret_cast<int *>(smem_raw);
  unsigned char *uni = smem_raw + (((size_t)sizeof(int) * SA_Q * S1 + 15) & ~(size_t)15);
  float4 *tile0 = reinterpret_cast<float4 *>(uni);
  float *gtile = reinterpret_cast<float *>(uni);

  const int tid = threadIdx.x, lane = tid & 31, part = tid >> 5;
  const int chunks = (M + SA_Q - 1) / SA_Q;
  const int ctot = C + (use_xyz ? 3 : 0);
  const int64_t E = (int64_t)M * K;
  const float never = __int_as_float(0xff800000);

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int m0 = (int)(blk % chunks) * SA_Q;
    const int i = m0 + lane;
    const bool valid = i < M;
    const int nv = min(SA_Q, M - m0);
    float qx = 0.f, qy = 0.f, qz = 0.f;
    if (valid) {
      const float *q = centroids + b * 3 * (int64_t)M + (int64_t)i * cps;
      qx = q[0];
      qy = q[cpc];
      qz = q[2 * (int64_t)cpc];
    }
    if (part == 0) {
      scent[0][lane] = qx;
      scent[1][lane] = qy;
      scent[2][lane] = qz;
    }
    const float2 mx[1] = {make_float2(-2.f * qx, -2.f * qx)}, my[1] = {make_float2(-2.f * qy, -2.f * qy)},
                 mz[1] = {make_float2(-2.f * qz, -2.f * qz)};
    float thr[1] = {valid ? sweep_threshold(r2, sweep_qq(qx, qy, qz)) : never};
    int done = 0;                   // hits of this centroid in the tiles swept so far (same in every warp)
    int *row = sidx + lane * S1;    // its hit list, ascending point index
    const float *rb = points + b * 3 * (int64_t)N;
    const int ntiles = (N + SA_TILE - 1) / SA_TILE;

    // ---- phase A: ball query ----------------------------------------------------------------
    float4 nxt[PER];
    auto fetch = [&](int t0) {
#pragma unroll
      for (int p = 0; p < PER; ++p) {
        const int j = t0 + tid + p * THREADS;
        float4 v = make_float4(0.f, 0.f, 0.f, __int_as_float(0x7f800000));
        if (j < N) {
          const float *r = rb + (int64_t)j * pps;
          const float x = r[0], y = r[pcs], z = r[2 * (int64_t)pcs];
          v = make_float4(x, y, z, sweep_key_w(x, y, z));
        }
        nxt[p] = v;
      }
    };
    auto commit = [&](float4 *dst) {
#pragma unroll
      for (int p = 0; p < PER; ++p) sweep_store_key(dst, tid + p * THREADS, nxt[p].x, nxt[p].y, nxt[p].z, nxt[p].w);
    };
    if (ntiles > 0) {
      fetch(0);
      commit(tile0);
    }
    __syncthreads();
    // Every warp sweeps its slice of the tile and keeps the hits as a bit mask; the slices' counts
    // are exchanged at the tile's barrier, after which each thread knows where its hits belong in
    // the centroid's list (hits of earlier tiles + hits of lower slices) and writes them there:
    // ascending point order without a merge.  The block leaves the loop at the first barrier after
    // all its lists are full.
    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * SA_TILE + part * QK;
      const float4 *tl = tile0 + (t & 1) * SA_TILE + part * QK;
      if (t + 1 < ntiles) fetch((t + 1) * SA_TILE);
      unsigned long long mask = 0;
      int cnt = 0;
      const bool was_full = !valid || done >= K;
#pragma unroll 2
      for (int u0 = 0; u0 < QK; u0 += 8) {
        float2 a[4];
        if (__builtin_expect(sweep_group2<1, true>(tl + u0, mx, my, mz, thr, a), 0)) {
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float av = (u & 1) ? a[u >> 1].y : a[u >> 1].x;
            if (!(av >= thr[0])) {  // padding keys carry +inf; a full row has thr = -inf
              const float4 r = sweep_load_key(tl, u0 + u);
              const float d = sqdist<float>(r.x, r.y, r.z, qx, qy, qz);
              if (d < r2) {
                mask |= 1ull << (u0 + u);
                if (done + ++cnt >= K) thr[0] = never;
              }
            }
          }
        }
      }
      tcount[t & 1][part][lane] = cnt;
      if (t + 1 < ntiles) commit(tile0 + ((t + 1) & 1) * SA_TILE);
      if (__syncthreads_and(was_full)) break;
      int before = 0, total = 0;
#pragma unroll
      for (int sp = 0; sp < SPLIT; ++sp) {
        const int c = tcount[t & 1][sp][lane];
        if (sp < part) before += c;
        total += c;
      }
      int pos = done + before;
      while (mask != 0 && pos < K) {
        const int bit = __ffsll((long long)mask) - 1;
        mask &= mask - 1;
        row[pos++] = t0 + bit;
      }
      done += total;
      if (done >= K) thr[0] = never;
    }
    __syncthreads();  // the lists' first entries are visible to every warp
    if (done < K) {   // short lists repeat their first hit; empty ones (and padding lanes) hold -1
      const int first = valid && done > 0 ? row[0] : -1;
      for (int c = (valid ? done : 0) + part; c < K; c += SPLIT) row[c] = first;
      if (part == 0 && valid && done == 0 && status) atomicOr(status, 1);
    }
    __syncthreads();  // lists complete; tiles and hit lists are dead from here on

    // ---- phase B: gather ----------------------------------------------------------------------
    const int ne = nv * K;                 // entries of this block, contiguous in the output
    const int64_t e_blk = (int64_t)m0 * K;
    float *ob = out + b * ctot * E + e_blk;
    if (index32) {
      int32_t *ip = index32 + b * E + e_blk;
      for (int e = tid; e < ne; e += THREADS) ip[e] = sidx[(e / K) * S1 + (e % K)];
    }
    if (use_xyz) {
      float *ox = ob + (int64_t)C * E;
      for (int e = tid; e < ne; e += THREADS) {
        const int c = e / K;
        const int id = sidx[c * S1 + (e - c * K)];
        float x = 0.f, y = 0.f, z = 0.f;
        if (id >= 0) {
          const float *r = rb + (int64_t)id * pps;
          x = __ldg(r);
          y = __ldg(r + pcs);
          z = __ldg(r + 2 * (int64_t)pcs);
        }
        __stcs(ox + e, __fsub_rn(x, scent[0][c]));
        __stcs(ox + E + e, __fsub_rn(y, scent[1][c]));
        __stcs(ox + 2 * E + e, __fsub_rn(z, scent[2][c]));
      }
    }
    if (C > 0) {
      const float *fb = featT + b * (int64_t)N * C;
      for (int s0 = 0; s0 < ne; s0 += SA_TE) {
        const int n = min(SA_TE, ne - s0);
        if (vec) {
          const int L = C >> 2;
          const float4 *fb4 = reinterpret_cast<const float4 *>(fb);
          // four entries per warp and step (lane = 8 * el + ql), as in gather_rows_vec4_kernel:
          // the 32 scalar stores of one instruction fall into 32 different banks.  A warp's steps
          // (entry group, block of eight row pieces) are taken four at a time to keep four loads
          // in flight per lane.
          const int ql = lane & 7, el = lane >> 3;
          constexpr int NW = THREADS / 32;
          const int QB = (L + 7) >> 3;
          const int ng = n >> 2;
          const int steps = ng > part ? ((ng - part + NW - 1) / NW) * QB : 0;
          int gi = part, qb = 0;
          for (int t = 0; t < steps; t += 4) {
            float4 v[4];
            int gg[4], qq[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              gg[w] = gi;
              qq[w] = 8 * qb + ql;
              v[w] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (t + w < steps && qq[w] < L) {
                const int g = s0 + 4 * gi + el;
                const int c = g / K;
                const int id = sidx[c * S1 + (g - c * K)];
                if (id >= 0) v[w] = __ldg(fb4 + (int64_t)id * L + qq[w]);
              }
              if (++qb == QB) {
                qb = 0;
                gi += NW;
              }
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              if (t + w < steps && qq[w] < L) {
                float *dst = gtile + (4 * qq[w]) * SA_TE + (((gg[w] ^ qq[w]) & (SA_TE / 4 - 1)) << 2) + el;
                dst[0] = v[w].x;
                dst[SA_TE] = v[w].y;
                dst[2 * SA_TE] = v[w].z;
                dst[3 * SA_TE] = v[w].w;
              }
            }
          }
          __syncthreads();
          const int nchunks = n >> 2;
          for (int u = tid; u < C * (SA_TE / 4); u += THREADS) {
            const int c = u >> 4, ch = u & 15;
            if (ch < nchunks) {
              const float4 v = *reinterpret_cast<const float4 *>(gtile + c * SA_TE + (((ch ^ (c >> 2)) & 15) << 2));
              __stcs(reinterpret_cast<float4 *>(ob + (int64_t)c * E + s0 + 4 * ch), v);
            }
          }
        } else {
          constexpr int S = SA_TE + 1;
          for (int e = part; e < n; e += THREADS / 32) {
            const int g = s0 + e;
            const int c0 = g / K;
            const int id = sidx[c0 * S1 + (g - c0 * K)];
            const float *row = fb + (int64_t)(id < 0 ? 0 : id) * C;
            for (int c = lane; c < C; c += 32) gtile[c * S + e] = id < 0 ? 0.f : __ldg(row + c);
          }
          __syncthreads();
          for (int c = part; c < C; c += THREADS / 32)
            for (int e = lane; e < n; e += 32) __stcs(ob + (int64_t)c * E + s0 + e, gtile[c * S + e]);
        }
        __syncthreads();
      }
    }
    __syncthreads();
  }
}

// Backward of the three coordinate channels: one warp per (cloud, centroid), lanes over K.
//   grad_points[b, index, d]  += g[b, C+d, m, k]
//   grad_centroids[b, m, d]   -= sum_k g[b, C+d, m, k]
__global__ void __launch_bounds__(256)
sa_group_bwd_xyz_kernel(const float *__restrict__ gout, const int32_t *__restrict__ index32, int64_t B, int C, int N,
                        int M, int K, int pps, int pcs, int cps, int cpc, float *__restrict__ gpoints,
                        float *__restrict__ gcent) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t E = (int64_t)M * K;
  for (int64_t w = warp; w < B * M; w += nwarps) {
    const int64_t b = w / M;
    const int m = (int)(w - b * M);
    const float *g = gout + (b * (C + 3) + C) * E + (int64_t)m * K;
    const int32_t *ip = index32 + b * E + (int64_t)m * K;
    float sx = 0.f, sy = 0.f, sz = 0.f;
    for (int k = lane; k < K; k += 32) {
      const float gx = g[k], gy = g[E + k], gz = g[2 * E + k];
      sx += gx;
      sy += gy;
      sz += gz;
      const int id = ip[k];
      if (id >= 0 && id < N && gpoints) {
        float *p = gpoints + b * 3 * (int64_t)N + (int64_t)id * pps;
        atomicAdd(p, gx);
        atomicAdd(p + pcs, gy);
        atomicAdd(p + 2 * (int64_t)pcs, gz);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sx += __shfl_xor_sync(0xffffffffu, sx, o);
      sy += __shfl_xor_sync(0xffffffffu, sy, o);
      sz += __shfl_xor_sync(0xffffffffu, sz, o);
    }
    if (lane == 0 && gcent) {
      float *c = gcent + b * 3 * (int64_t)M + (int64_t)m * cps;
      c[0] = -sx;
      c[cpc] = -sy;
      c[2 * (int64_t)cpc] = -sz;
    }
  }
}

bool sa_shape_ok(int64_t B, int64_t C, int64_t N, int64_t M, int64_t K) {
  return B >= 0 && B <= 65535 && C >= 0 && C <= ROWS_MAX_C && N >= 0 && N < (1LL << 30) && M >= 0 &&
         M < (1LL << 30) && K >= 1 && K <= SA_MAX_K && M * K < (1LL << 31);
}

}  // namespace
}  // namespace tk3d

using namespace tk3d;

extern "C" int tk3d_sa_group_supported(int64_t B, int64_t C, int64_t N, int64_t M, int64_t K, int dtype) {
  return dtype == TK3D_F32 && sa_shape_ok(B, C, N, M, K) ? 1 : 0;
}

extern "C" size_t tk3d_sa_group_scratch_bytes(int64_t B, int64_t C, int64_t N, int64_t M, int64_t K, int dtype) {
  if (!tk3d_sa_group_supported(B, C, N, M, K, dtype) || C == 0) return 0;
  return rows_scratch_bytes(B, C, N);
}

extern "C" int tk3d_sa_group_fwd(const void *points, const void *centroids, const void *feature, int64_t B, int64_t C,
                                 int64_t N, int64_t M, float radius, int64_t K, int xyz_channel_first, int use_xyz,
                                 void *out, int32_t *index32, int32_t *status, void *scratch, size_t scratch_bytes,
                                 int dtype, void *stream) {
  TK3D_RANGE("tk3d_sa_group_fwd");
  TK3D_REQUIRE(dtype == TK3D_F32, TK3D_ERR_DTYPE, "sa_group_fwd: only fp32 has a fused path (dtype %d)", dtype);
  TK3D_REQUIRE(sa_shape_ok(B, C, N, M, K), TK3D_ERR_SHAPE,
               "sa_group_fwd: unsupported shape B=%lld C=%lld N=%lld M=%lld K=%lld (C <= %d, 1 <= K <= %d)",
               (long long)B, (long long)C, (long long)N, (long long)M, (long long)K, ROWS_MAX_C, SA_MAX_K);
  const int ctot = (int)C + (use_xyz ? 3 : 0);
  if (B * M * ctot == 0) return TK3D_OK;
  TK3D_REQUIRE(centroids && out && (points || N == 0) && (feature || C == 0), TK3D_ERR_NULL,
               "sa_group_fwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  const float *featT = nullptr;
  if (C > 0 && N > 0) {
    const size_t want = rows_scratch_bytes(B, C, N);
    TK3D_REQUIRE(scratch != nullptr && scratch_bytes >= want, TK3D_ERR_SCRATCH,
                 "sa_group_fwd: scratch of %zu bytes required (got %zu)", want, scratch_bytes);
    int rc = transpose_bcn((const float *)feature, (float *)scratch, B, C, N, st);
    if (rc) return rc;
    featT = (const float *)scratch;
  }
  const int vec = C > 0 && C % 4 == 0 && K % 4 == 0 &&
                  ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scratch)) & 15) == 0;
  const SaSmem sm = sa_smem((int)C, (int)K, vec);
  const int64_t total = B * ((M + SA_Q - 1) / SA_Q);
  const bool wide = total <= 2 * (int64_t)sm_count();  // few blocks: eight warps per 32 centroids
  if (sm.total > 48 * 1024)
    TK3D_CUDA(raise_smem_limit(wide ? (const void *)sa_group_fwd_kernel<8> : (const void *)sa_group_fwd_kernel<4>,
                               (int)sm.total));
  const int64_t cap = (int64_t)sm_count() * 64;
  const float r2 = radius * radius;
  const int pps = xyz_channel_first ? 1 : 3, pcs = xyz_channel_first ? (int)N : 1;
  const int cps = xyz_channel_first ? 1 : 3, cpc = xyz_channel_first ? (int)M : 1;
  const unsigned grid = (unsigned)(total < cap ? total : cap);
  if (wide)
    sa_group_fwd_kernel<8><<<grid, 256, sm.total, st>>>(
        (const float *)points, (const float *)centroids, featT, B, (int)C, (int)N, (int)M, pps, pcs, cps, cpc, r2,
        (int)K, use_xyz ? 1 : 0, vec, (float *)out, index32, status, total);
  else
    sa_group_fwd_kernel<4><<<grid, 128, sm.total, st>>>(
        (const float *)points, (const float *)centroids, featT, B, (int)C, (int)N, (int)M, pps, pcs, cps, cpc, r2,
        (int)K, use_xyz ? 1 : 0, vec, (float *)out, index32, status, total);
  return check_launch("sa_group_fwd_kernel");
}

namespace tk3d {
namespace {

// Feature gradient without the row path (C or K not a multiple of 4): one thread per gradient element.
__global__ void __launch_bounds__(256)
sa_group_bwd_feat_kernel(const float *__restrict__ gout, const int32_t *__restrict__ index32, int64_t B, int C, int N,
                         int64_t E, int64_t gstride, float *__restrict__ gfeat, int32_t *__restrict__ status) {
  const int64_t total = B * C * E;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = t % E;
    const int64_t bc = t / E;
    const int64_t b = bc / C;
    const int c = (int)(bc - b * C);
    const int id = index32[b * E + e];
    if (id < 0 || id >= N) {
      if (status) atomicOr(status, 1);
      continue;
    }
    atomicAdd(gfeat + (b * C + c) * (int64_t)N + id, gout[b * gstride + (int64_t)c * E + e]);
  }
}

}  // namespace
}  // namespace tk3d

extern "C" int tk3d_sa_group_bwd(const void *gout, const int32_t *index32, int64_t B, int64_t C, int64_t N, int64_t M,
                                 int64_t K, int xyz_channel_first, int use_xyz, void *gfeature, void *gpoints,
                                 void *gcentroids, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                                 void *stream) {
  TK3D_RANGE("tk3d_sa_group_bwd");
  TK3D_REQUIRE(dtype == TK3D_F32, TK3D_ERR_DTYPE, "sa_group_bwd: only fp32 has a fused path (dtype %d)", dtype);
  TK3D_REQUIRE(sa_shape_ok(B, C, N, M, K), TK3D_ERR_SHAPE, "sa_group_bwd: unsupported shape");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t E = M * K;
  const int64_t ctot = C + (use_xyz ? 3 : 0);
  const int64_t gstride = ctot * E;
  TK3D_REQUIRE(B * E == 0 || (gout && index32), TK3D_ERR_NULL, "sa_group_bwd: a pointer is NULL");
  if (gfeature && B * C * N > 0) {
    const bool vec = C % 4 == 0 && K % 4 == 0 && C >= 4 && (N + 31) / 32 <= 65535 && scratch != nullptr &&
                     scratch_bytes >= rows_scratch_bytes(B, C, N) &&
                     ((reinterpret_cast<uintptr_t>(gout) | reinterpret_cast<uintptr_t>(scratch)) & 15) == 0;
    if (vec) {
      TK3D_CUDA(cudaMemsetAsync(scratch, 0, rows_scratch_bytes(B, C, N), st));
      if (E > 0) {
        const size_t smem = (size_t)C * ROWS_TE * sizeof(float);
        if (smem > 48 * 1024)
          TK3D_CUDA(raise_smem_limit((const void *)scatter_rows_vec4_kernel<1, int32_t>, (int)smem));
        dim3 grid((unsigned)((E + ROWS_TE - 1) / ROWS_TE), (unsigned)B);
        scatter_rows_vec4_kernel<1, int32_t><<<grid, ROWS_THREADS, smem, st>>>(
            (const float *)gout, index32, nullptr, (int)C, N, E, gstride, (float *)scratch, status);
        int rc = check_launch("scatter_rows_vec4_kernel");
        if (rc) return rc;
      }
      int rc = transpose_bcn((const float *)scratch, (float *)gfeature, B, N, C, st);
      if (rc) return rc;
    } else {
      TK3D_CUDA(cudaMemsetAsync(gfeature, 0, sizeof(float) * (size_t)(B * C * N), st));
      if (E > 0) {
        const int64_t blocks = (B * C * E + 255) / 256, cap = (int64_t)sm_count() * 32;
        sa_group_bwd_feat_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(
            (const float *)gout, index32, B, (int)C, (int)N, E, gstride, (float *)gfeature, status);
        int rc = check_launch("sa_group_bwd_feat_kernel");
        if (rc) return rc;
      }
    }
  }
  if (use_xyz && (gpoints || gcentroids)) {
    if (gpoints && B * N > 0) TK3D_CUDA(cudaMemsetAsync(gpoints, 0, sizeof(float) * (size_t)(B * N * 3), st));
    if (B * M > 0) {
      const int pps = xyz_channel_first ? 1 : 3, pcs = xyz_channel_first ? (int)N : 1;
      const int cps = xyz_channel_first ? 1 : 3, cpc = xyz_channel_first ? (int)M : 1;
      const int64_t blocks = (B * M + 7) / 8, cap = (int64_t)sm_count() * 32;
      sa_group_bwd_xyz_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(
          (const float *)gout, index32, B, (int)C, (int)N, (int)M, (int)K, pps, pcs, cps, cpc, (float *)gpoints,
          (float *)gcentroids);
      int rc = check_launch("sa_group_bwd_xyz_kernel");
      if (rc) return rc;
    }
  }
  return TK3D_OK;
}

TK3D_BOUNDS_TU(sa_group)
