// Ball query: first k key indices (ascending) whose squared distance is < radius^2.
//
// fp32: the filter-then-verify sweep of sweep.cuh (pair layout, packed FMAs) with a constant
// bound (radius^2).  With many queries one thread serves a query and writes verified hits straight
// to the output row; with few, several warps share 32 queries and place their hits by counting
// (ball_query_split_kernel below).  A query stops testing once it has k hits (its threshold becomes
// -inf) and a block leaves the key loop as soon as all its queries are full -- the reference keeps
// scanning to the end of the cloud.  Short rows are padded with the first hit, rows without a hit
// are filled with -1, so every output element is written here.
#include "sweep.cuh"

namespace tk3d {

namespace {

constexpr int BQ_THREADS = 128;
constexpr int BQ_TILE = 512;

__global__ void __launch_bounds__(BQ_THREADS)
ball_query_fast_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2,
                       float r2, int k, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  constexpr int PER = BQ_TILE / BQ_THREADS;
  __shared__ float4 tile[2][BQ_TILE];
  const int tid = threadIdx.x;
  const int chunks = (N1 + BQ_THREADS - 1) / BQ_THREADS;

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int i = (int)(blk % chunks) * BQ_THREADS + tid;
    const bool valid = i < N1;
    float qx = 0.f, qy = 0.f, qz = 0.f;
    if (valid) load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx, qy, qz);
    const float2 mx[1] = {make_float2(-2.f * qx, -2.f * qx)}, my[1] = {make_float2(-2.f * qy, -2.f * qy)},
                 mz[1] = {make_float2(-2.f * qz, -2.f * qz)};
    const float never = __int_as_float(0xff800000);
    float thr[1] = {valid ? sweep_threshold(r2, sweep_qq(qx, qy, qz)) : never};
    int cnt = 0;
    int64_t first = -1;
    const int64_t row = (b * N1 + (valid ? i : 0)) * (int64_t)k;  // offset of this query's output row

    const float *rb = key + b * (int64_t)N2 * 3;
    const int ntiles = (N2 + BQ_TILE - 1) / BQ_TILE;
#pragma unroll
    for (int p = 0; p < PER; ++p) {
      const int u = tid + p * BQ_THREADS;
      float4 v = make_float4(0.f, 0.f, 0.f, __int_as_float(0x7f800000));
      if (u < N2) {
        float x, y, z;
        load_xyz(rb, u, kl, x, y, z);
        v = make_float4(x, y, z, sweep_key_w(x, y, z));
      }
      sweep_store_key(tile[0], u, v.x, v.y, v.z, v.w);
    }
    __syncthreads();

    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * BQ_TILE;
      const float4 *tl = tile[t & 1];
      const bool more = t + 1 < ntiles;
      float4 nxt[PER];
      if (more) {
#pragma unroll
        for (int p = 0; p < PER; ++p) {
          const int j = t0 + BQ_TILE + tid + p * BQ_THREADS;
          float4 v = make_float4(0.f, 0.f, 0.f, __int_as_float(0x7f800000));
          if (j < N2) {
            float x, y, z;
            load_xyz(rb, j, kl, x, y, z);
            v = make_float4(x, y, z, sweep_key_w(x, y, z));
          }
          nxt[p] = v;
        }
      }
      const int lim = (min(BQ_TILE, N2 - t0) + 7) & ~7;
#pragma unroll 2
      for (int u0 = 0; u0 < lim; u0 += 8) {
        float2 a[4];
        if (__builtin_expect(sweep_group2<1, true>(tl + u0, mx, my, mz, thr, a), 0)) {
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int j = t0 + u0 + u;
            const float av = (u & 1) ? a[u >> 1].y : a[u >> 1].x;
            if (!(av >= thr[0])) {  // padding keys carry +inf; a full row has thr = -inf
              const float4 r = sweep_load_key(tl, u0 + u);
              const float d = sqdist<float>(r.x, r.y, r.z, qx, qy, qz);
              if (d < r2) {
                index.put(row + cnt, j);
                if (cnt == 0) first = j;
                if (++cnt == k) thr[0] = never;
              }
            }
          }
        }
      }
      if (more) {
        float4 *nx = tile[(t + 1) & 1];
#pragma unroll
        for (int p = 0; p < PER; ++p) sweep_store_key(nx, tid + p * BQ_THREADS, nxt[p].x, nxt[p].y, nxt[p].z, nxt[p].w);
      }
      // One barrier per tile; it also votes on "every query of this block is complete".
      if (__syncthreads_and(!valid || cnt == k)) break;
    }
    if (valid)
      for (int c = cnt; c < k; ++c) index.put(row + c, first);
    __syncthreads();
  }
}

// Few queries (B*N1 below a few hundred thousand): one query per thread cannot fill 148 SMs.  Here a
// block of SPLIT warps serves 32 queries (lane = query) and warp s sweeps the s-th slice of every
// 256-key tile, so SPLIT times as many warps are in flight.  A thread records the hits of its slice
// as a bit mask (at most 64 keys), the slices' hit counts of the tile are exchanged through shared
// memory at the tile's barrier, and every thread then knows where its hits belong in the query's
// row (hits of earlier tiles + hits of lower slices of this tile) and writes them there: rows come
// out in ascending key order without a merge, for any K.  A query with K hits stops testing, and
// the block leaves the key loop at the first barrier after all its queries are full.
constexpr int BS_TILE = 256;

template <int SPLIT>
__global__ void __launch_bounds__(32 * SPLIT)
ball_query_split_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2,
                        float r2, int k, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  constexpr int THREADS = 32 * SPLIT;
  constexpr int PER = BS_TILE / THREADS;
  constexpr int QK = BS_TILE / SPLIT;  // keys per warp per tile (64 or 32)
  static_assert(PER >= 1 && QK <= 64 && QK % 8 == 0, "slice must fit a 64-bit hit mask");
  __shared__ float4 tile[2][BS_TILE];
  __shared__ int tcount[2][SPLIT][32];
  const int tid = threadIdx.x, lane = tid & 31, part = tid >> 5;
  const int chunks = (N1 + 31) / 32;
  const float never = __int_as_float(0xff800000);

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int i = (int)(blk % chunks) * 32 + lane;
    const bool valid = i < N1;
    float qx = 0.f, qy = 0.f, qz = 0.f;
    if (valid) load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx, qy, qz);
    const float2 mx[1] = {make_float2(-2.f * qx, -2.f * qx)}, my[1] = {make_float2(-2.f * qy, -2.f * qy)},
                 mz[1] = {make_float2(-2.f * qz, -2.f * qz)};
    const float open_thr = sweep_threshold(r2, sweep_qq(qx, qy, qz));
    float thr[1] = {valid ? open_thr : never};
    const int64_t row = (b * N1 + (valid ? i : 0)) * (int64_t)k;
    int done = 0;  // hits of this query in the tiles swept so far (the same number in every warp)
    const float *rb = key + b * (int64_t)N2 * 3;
    const int ntiles = (N2 + BS_TILE - 1) / BS_TILE;

    float4 nxt[PER];
    auto fetch = [&](int t0) {
#pragma unroll
      for (int p = 0; p < PER; ++p) {
        const int j = t0 + tid + p * THREADS;
        float4 v = make_float4(0.f, 0.f, 0.f, __int_as_float(0x7f800000));
        if (j < N2) {
          float x, y, z;
          load_xyz(rb, j, kl, x, y, z);
          v = make_float4(x, y, z, sweep_key_w(x, y, z));
        }
        nxt[p] = v;
      }
    };
    auto commit = [&](float4 *dst) {
#pragma unroll
      for (int p = 0; p < PER; ++p) sweep_store_key(dst, tid + p * THREADS, nxt[p].x, nxt[p].y, nxt[p].z, nxt[p].w);
    };
    fetch(0);
    commit(tile[0]);
    __syncthreads();
    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * BS_TILE + part * QK;
      const float4 *tl = tile[t & 1] + part * QK;
      if (t + 1 < ntiles) fetch((t + 1) * BS_TILE);
      unsigned long long mask = 0;
      int cnt = 0;
      const bool was_full = !valid || done >= k;
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
                if (done + ++cnt >= k) thr[0] = never;  // whatever the lower slices found, this row is full
              }
            }
          }
        }
      }
      tcount[t & 1][part][lane] = cnt;
      if (t + 1 < ntiles) commit(tile[(t + 1) & 1]);
      // One barrier per tile; it also votes on "every query of this block was full before this tile"
      // (such a tile recorded no hit anywhere, so nothing is left to write).
      if (__syncthreads_and(was_full)) break;
      int before = 0, total = 0;
#pragma unroll
      for (int s = 0; s < SPLIT; ++s) {
        const int c = tcount[t & 1][s][lane];
        if (s < part) before += c;
        total += c;
      }
      int pos = done + before;
      while (mask != 0 && pos < k) {
        const int bit = __ffsll((long long)mask) - 1;
        mask &= mask - 1;
        index.put(row + pos, t0 + bit);
        ++pos;
      }
      done += total;
      if (done >= k) thr[0] = never;
    }
    __syncthreads();  // the row's first entry, written by whichever warp found it, is visible now
    if (valid && done < k) {
      const int64_t first = done > 0 ? index.get(row) : -1;
      for (int c = done + part; c < k; c += SPLIT) index.put(row + c, first);
    }
    __syncthreads();
  }
}

// The same scheme with the plain distance test on every key (float64, whose inputs the packed
// float32 filter cannot serve): SPLIT warps per 32 queries, hit masks, positional writes.
template <typename T, int SPLIT>
__global__ void __launch_bounds__(32 * SPLIT)
ball_query_split_exact_kernel(const T *__restrict__ query, const T *__restrict__ key, int64_t B, int N1, int N2, T r2,
                              int k, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  constexpr int THREADS = 32 * SPLIT;
  constexpr int PER = BS_TILE / THREADS;
  constexpr int QK = BS_TILE / SPLIT;
  __shared__ T sx[2][BS_TILE], sy[2][BS_TILE], sz[2][BS_TILE];
  __shared__ int tcount[2][SPLIT][32];
  const int tid = threadIdx.x, lane = tid & 31, part = tid >> 5;
  const int chunks = (N1 + 31) / 32;

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int i = (int)(blk % chunks) * 32 + lane;
    const bool valid = i < N1;
    T qx = 0, qy = 0, qz = 0;
    if (valid) load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx, qy, qz);
    const int64_t row = (b * N1 + (valid ? i : 0)) * (int64_t)k;
    int done = 0;
    const T *rb = key + b * (int64_t)N2 * 3;
    const int ntiles = (N2 + BS_TILE - 1) / BS_TILE;

    T nx[PER], ny[PER], nz[PER];
    auto fetch = [&](int t0) {
#pragma unroll
      for (int p = 0; p < PER; ++p) {
        const int j = t0 + tid + p * THREADS;
        nx[p] = ny[p] = nz[p] = 0;
        if (j < N2) load_xyz(rb, j, kl, nx[p], ny[p], nz[p]);
      }
    };
    auto commit = [&](int buf) {
#pragma unroll
      for (int p = 0; p < PER; ++p) {
        sx[buf][tid + p * THREADS] = nx[p];
        sy[buf][tid + p * THREADS] = ny[p];
        sz[buf][tid + p * THREADS] = nz[p];
      }
    };
    fetch(0);
    commit(0);
    __syncthreads();
    for (int t = 0; t < ntiles; ++t) {
      const int buf = t & 1;
      const int u_lo = part * QK;
      const int t0 = t * BS_TILE + u_lo;
      if (t + 1 < ntiles) fetch((t + 1) * BS_TILE);
      unsigned long long mask = 0;
      int cnt = 0;
      const bool was_full = !valid || done >= k;
      const int lim = min(QK, N2 - t0);  // may be <= 0 in the last tile
      if (!was_full) {
        for (int u = 0; u < lim; ++u) {
          const T d = sqdist<T>(sx[buf][u_lo + u], sy[buf][u_lo + u], sz[buf][u_lo + u], qx, qy, qz);
          if (d < r2) {
            mask |= 1ull << u;
            if (done + ++cnt >= k) break;
          }
        }
      }
      tcount[buf][part][lane] = cnt;
      if (t + 1 < ntiles) commit(buf ^ 1);
      if (__syncthreads_and(was_full)) break;
      int before = 0, total = 0;
#pragma unroll
      for (int s = 0; s < SPLIT; ++s) {
        const int c = tcount[buf][s][lane];
        if (s < part) before += c;
        total += c;
      }
      int pos = done + before;
      while (mask != 0 && pos < k) {
        const int bit = __ffsll((long long)mask) - 1;
        mask &= mask - 1;
        index.put(row + pos, t0 + bit);
        ++pos;
      }
      done += total;
    }
    __syncthreads();
    if (valid && done < k) {
      const int64_t first = done > 0 ? index.get(row) : -1;
      for (int c = done + part; c < k; c += SPLIT) index.put(row + c, first);
    }
    __syncthreads();
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
ball_query_generic_kernel(const T *__restrict__ query, const T *__restrict__ key, int64_t B, int64_t N1, int64_t N2,
                          T r2, int64_t k, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  constexpr int TILE = 256;
  __shared__ T sx[TILE], sy[TILE], sz[TILE];
  const int tid = threadIdx.x;
  const int64_t chunks = (N1 + TILE - 1) / TILE;
  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int64_t i = (blk % chunks) * TILE + tid;
    const bool valid = i < N1;
    T qx = 0, qy = 0, qz = 0;
    if (valid) load_xyz(query + b * 3 * N1, i, ql, qx, qy, qz);
    const int64_t row = (b * N1 + (valid ? i : 0)) * k;
    int64_t cnt = 0, first = -1;
    const T *rb = key + b * N2 * 3;
    for (int64_t t0 = 0; t0 < N2; t0 += TILE) {
      const int64_t jl = t0 + tid;
      if (jl < N2) load_xyz(rb, jl, kl, sx[tid], sy[tid], sz[tid]);
      __syncthreads();
      const int lim = (int)((N2 - t0) < TILE ? (N2 - t0) : TILE);
      if (valid && cnt < k) {
        for (int u = 0; u < lim && cnt < k; ++u) {
          const T d = sqdist<T>(sx[u], sy[u], sz[u], qx, qy, qz);
          if (d < r2) {
            index.put(row + cnt, t0 + u);
            if (cnt == 0) first = t0 + u;
            ++cnt;
          }
        }
      }
      if (__syncthreads_and(!valid || cnt == k)) break;
    }
    if (valid)
      for (int64_t c = cnt; c < k; ++c) index.put(row + c, first);
    __syncthreads();
  }
}

}  // namespace
}  // namespace tk3d

using namespace tk3d;

static int ball_query_impl(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, float radius,
                           int64_t k, int channel_first, void *index, int index32, int dtype, void *stream) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "ball_query: dtype %d", dtype);
  TK3D_REQUIRE(B >= 0 && N1 >= 0 && N2 >= 0, TK3D_ERR_SHAPE, "ball_query: negative size");
  TK3D_REQUIRE(k >= 1 && k < (1LL << 31), TK3D_ERR_K, "ball_query: max_neighbors must be >= 1 (got %lld)",
               (long long)k);
  TK3D_REQUIRE(N1 < (1LL << 30) && N2 < (1LL << 30), TK3D_ERR_SHAPE, "ball_query: clouds limited to 2^30 points");
  if (B * N1 == 0) return TK3D_OK;
  TK3D_REQUIRE(query && index && (key || N2 == 0), TK3D_ERR_NULL, "ball_query: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  const XyzLayout ql = xyz_layout(channel_first, N1), kl = xyz_layout(channel_first, N2);
  const IndexOut io = index_out(index, index32, B * N1 * k);
  if (dtype == TK3D_F32) {
    const float r2 = radius * radius;  // squared in fp32, as the reference does for float tensors
    const int64_t cap = (int64_t)sm_count() * 256;
    if (B * N1 < (int64_t)sm_count() * 16 * BQ_THREADS) {
      const int64_t total = B * ((N1 + 31) / 32);
      const unsigned grid = (unsigned)(total < cap ? total : cap);
      if (total <= 2 * (int64_t)sm_count())  // very few queries: eight warps per 32 queries
        ball_query_split_kernel<8><<<grid, 256, 0, st>>>((const float *)query, (const float *)key, B, (int)N1, (int)N2,
                                                         r2, (int)k, io, total, ql, kl);
      else
        ball_query_split_kernel<4><<<grid, 128, 0, st>>>((const float *)query, (const float *)key, B, (int)N1, (int)N2,
                                                         r2, (int)k, io, total, ql, kl);
      return check_launch("ball_query_split_kernel");
    }
    const int64_t total = B * ((N1 + BQ_THREADS - 1) / BQ_THREADS);
    ball_query_fast_kernel<<<(unsigned)(total < cap ? total : cap), BQ_THREADS, 0, st>>>(
        (const float *)query, (const float *)key, B, (int)N1, (int)N2, r2, (int)k, io, total, ql, kl);
    return check_launch("ball_query_fast_kernel");
  }
  const double r = (double)radius;
  if (B * N1 < (int64_t)sm_count() * 8 * 256) {  // too few queries for one thread each
    const int64_t tot = B * ((N1 + 31) / 32);
    const int64_t cap4 = (int64_t)sm_count() * 64;
    ball_query_split_exact_kernel<double, 4><<<(unsigned)(tot < cap4 ? tot : cap4), 128, 0, st>>>(
        (const double *)query, (const double *)key, B, (int)N1, (int)N2, r * r, (int)k, io, tot, ql, kl);
    return check_launch("ball_query_split_exact_kernel");
  }
  const int64_t total = B * ((N1 + 255) / 256);
  const int64_t cap = (int64_t)sm_count() * 64;
  ball_query_generic_kernel<double><<<(unsigned)(total < cap ? total : cap), 256, 0, st>>>(
      (const double *)query, (const double *)key, B, N1, N2, r * r, k, io, total, ql, kl);
  return check_launch("ball_query_generic_kernel");
}

extern "C" int tk3d_ball_query(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, float radius,
                               int64_t k, int64_t *index, int dtype, void *stream) {
  TK3D_RANGE("tk3d_ball_query");
  return ball_query_impl(query, key, B, N1, N2, radius, k, 0, index, 0, dtype, stream);
}

extern "C" int tk3d_ball_query_layout(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2,
                                      float radius, int64_t k, int xyz_channel_first, void *index, int index_dtype,
                                      int dtype, void *stream) {
  TK3D_RANGE("tk3d_ball_query_layout");
  TK3D_REQUIRE(index_dtype == TK3D_I64 || index_dtype == TK3D_I32, TK3D_ERR_DTYPE, "ball_query: index_dtype %d",
               index_dtype);
  return ball_query_impl(query, key, B, N1, N2, radius, k, xyz_channel_first != 0, index, index_dtype == TK3D_I32,
                         dtype, stream);
}

TK3D_BOUNDS_TU(ball_query)
