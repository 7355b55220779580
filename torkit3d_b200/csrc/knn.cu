// Brute-force k nearest neighbours (squared distances, rows sorted ascending by (distance, index)).
//
// Three kernels:
//   knn_small_kernel<K,Q>  fp32, k <= 4: per-thread top-K in registers, filter-then-verify sweep
//                          (sweep.cuh), insertion straight from the verify branch.  With k << N2
//                          the branch is rare (about k ln(N2/k) times per query).
//   knn_buffered_kernel<Q> fp32, 4 < k <= 128: same filter, but passing keys are only appended
//                          (predicated store, no branch) to a small per-query candidate buffer in
//                          shared memory; buffers are drained into per-query sorted lists (also in
//                          shared memory) by the whole warp at once, when any lane's buffer is
//                          nearly full and at the end of every key tile.  This keeps the lanes of a
//                          warp in step even when k ln(N2/k) is not small against N2.
//   knn_generic_kernel<T>  any type / any k: one query per thread, exact distances, sorted list kept
//                          directly in the output rows.
// All of them take decisions on the exactly rounded distance and scan keys in ascending order with
// strict comparisons, so the retained set and its order are reproducible bit for bit.
#include "sweep.cuh"

namespace tk3d {

namespace {

constexpr int KN_THREADS = 128;
constexpr int KN_TILE = 256;
constexpr int KN_CAP = 16;   // candidate buffer entries per query
constexpr int KN_STEP = 8;   // keys processed between two buffer-occupancy checks

__device__ __forceinline__ float qnan() { return __int_as_float(0x7fc00000); }
__device__ __forceinline__ float pinf() { return __int_as_float(0x7f800000); }

// Stage one key tile (padded with points that can only reach the verify path, where they are
// rejected by index) from registers or global memory.
__device__ __forceinline__ float4 make_key(const float *__restrict__ rb, int j, int nr) {
  if (j < nr) {
    const float x = rb[(int64_t)j * 3 + 0], y = rb[(int64_t)j * 3 + 1], z = rb[(int64_t)j * 3 + 2];
    return make_float4(x, y, z, sweep_key_w(x, y, z));
  }
  return make_float4(0.f, 0.f, 0.f, pinf());
}

// ---------------------------------------------------------------------------------------------
template <int K, int Q>
__global__ void __launch_bounds__(KN_THREADS)
knn_small_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2,
                 float *__restrict__ dist, int64_t *__restrict__ index, int64_t blocks_total) {
  constexpr int TILE = 512, PER = TILE / KN_THREADS;
  constexpr int GK = 8 / Q;  // keys per filter group: eight (key, query) pairs share one branch
  __shared__ float4 tile[2][TILE];  // pair layout of sweep.cuh
  const int tid = threadIdx.x;
  const int chunks = (N1 + KN_THREADS * Q - 1) / (KN_THREADS * Q);

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int i0 = (int)(blk % chunks) * (KN_THREADS * Q) + tid;
    float qx[Q], qy[Q], qz[Q], thr[Q];
    float2 mx[Q], my[Q], mz[Q];
    float kd[Q][K];
    int ki[Q][K];
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = i0 + s * KN_THREADS;
      if (i < N1) {
        const float *q = query + (b * N1 + i) * 3;
        qx[s] = q[0];
        qy[s] = q[1];
        qz[s] = q[2];
        thr[s] = qnan();  // accept everything until the list is full
      } else {
        qx[s] = qy[s] = qz[s] = 0.f;
        thr[s] = -pinf();
      }
      mx[s] = make_float2(-2.f * qx[s], -2.f * qx[s]);
      my[s] = make_float2(-2.f * qy[s], -2.f * qy[s]);
      mz[s] = make_float2(-2.f * qz[s], -2.f * qz[s]);
#pragma unroll
      for (int c = 0; c < K; ++c) {
        kd[s][c] = pinf();
        ki[s][c] = 0x7fffffff;  // sentinel: orders after every real index
      }
    }

    const float *rb = key + b * (int64_t)N2 * 3;
    const int ntiles = (N2 + TILE - 1) / TILE;
#pragma unroll
    for (int p = 0; p < PER; ++p) {
      const int u = tid + p * KN_THREADS;
      const float4 v = make_key(rb, u, N2);
      sweep_store_key(tile[0], u, v.x, v.y, v.z, v.w);
    }
    __syncthreads();

    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * TILE;
      const float4 *tl = tile[t & 1];
      const bool more = t + 1 < ntiles;
      float4 nxt[PER];
      if (more) {
#pragma unroll
        for (int p = 0; p < PER; ++p) nxt[p] = make_key(rb, t0 + TILE + tid + p * KN_THREADS, N2);
      }
      const int lim = (min(TILE, N2 - t0) + GK - 1) / GK * GK;
#pragma unroll 2
      for (int u0 = 0; u0 < lim; u0 += GK) {
        float2 a[4];
        if (__builtin_expect(sweep_group2<Q>(tl + u0, mx, my, mz, thr, a), 0)) {
#pragma unroll
          for (int p = 0; p < GK / 2; ++p) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int j = t0 + u0 + 2 * p + h;
              if (j >= N2) continue;
              const float4 r = sweep_load_key(tl, u0 + 2 * p + h);
#pragma unroll
              for (int s = 0; s < Q; ++s) {
                const float av = h ? a[p * Q + s].y : a[p * Q + s].x;
                if (!(av >= thr[s])) {
                  const float d = sqdist<float>(r.x, r.y, r.z, qx[s], qy[s], qz[s]);
                  // (d, j) enters iff it orders before the current last entry; sentinels carry
                  // (+inf, INT_MAX) so real entries always precede them.
                  if (d < kd[s][K - 1] || (d == kd[s][K - 1] && j < ki[s][K - 1])) {
                    kd[s][K - 1] = d;
                    ki[s][K - 1] = j;
#pragma unroll
                    for (int c = K - 1; c > 0; --c) {
                      const bool lt =
                          kd[s][c] < kd[s][c - 1] || (kd[s][c] == kd[s][c - 1] && ki[s][c] < ki[s][c - 1]);
                      if (lt) {
                        const float td = kd[s][c];
                        kd[s][c] = kd[s][c - 1];
                        kd[s][c - 1] = td;
                        const int ti = ki[s][c];
                        ki[s][c] = ki[s][c - 1];
                        ki[s][c - 1] = ti;
                      }
                    }
                    if (ki[s][K - 1] != 0x7fffffff)
                      thr[s] = sweep_threshold(kd[s][K - 1], sweep_qq(qx[s], qy[s], qz[s]));
                  }
                }
              }
            }
          }
        }
      }
      if (more) {
        float4 *nx = tile[(t + 1) & 1];
#pragma unroll
        for (int p = 0; p < PER; ++p) sweep_store_key(nx, tid + p * KN_THREADS, nxt[p].x, nxt[p].y, nxt[p].z, nxt[p].w);
      }
      __syncthreads();
    }

#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = i0 + s * KN_THREADS;
      if (i < N1) {
        float *od = dist + (b * N1 + i) * K;
        int64_t *oi = index + (b * N1 + i) * K;
#pragma unroll
        for (int c = 0; c < K; ++c) {
          od[c] = kd[s][c];
          oi[c] = (int64_t)ki[s][c];
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
template <int Q>
__global__ void __launch_bounds__(KN_THREADS)
knn_buffered_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2,
                    int k, float *__restrict__ dist, int64_t *__restrict__ index, int64_t blocks_total) {
  constexpr int PER = KN_TILE / KN_THREADS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float4 *tile = reinterpret_cast<float4 *>(smem_raw);                        // [2][KN_TILE]
  float *ld = reinterpret_cast<float *>(tile + 2 * KN_TILE);                  // [Q][k][THREADS]
  int *li = reinterpret_cast<int *>(ld + (size_t)Q * k * KN_THREADS);         // [Q][k][THREADS]
  int *buf = li + (size_t)Q * k * KN_THREADS;                                 // [Q][CAP][THREADS]
  const int tid = threadIdx.x;
  const int chunks = (N1 + KN_THREADS * Q - 1) / (KN_THREADS * Q);

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int i0 = (int)(blk % chunks) * (KN_THREADS * Q) + tid;
    float qx[Q], qy[Q], qz[Q], mx[Q], my[Q], mz[Q], thr[Q];
    int cnt[Q], nk[Q];
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = i0 + s * KN_THREADS;
      if (i < N1) {
        const float *q = query + (b * N1 + i) * 3;
        qx[s] = q[0];
        qy[s] = q[1];
        qz[s] = q[2];
        thr[s] = qnan();
      } else {
        qx[s] = qy[s] = qz[s] = 0.f;
        thr[s] = -pinf();
      }
      mx[s] = -2.f * qx[s];
      my[s] = -2.f * qy[s];
      mz[s] = -2.f * qz[s];
      cnt[s] = 0;
      nk[s] = 0;
    }

    const float *rb = key + b * (int64_t)N2 * 3;
    const int ntiles = (N2 + KN_TILE - 1) / KN_TILE;
#pragma unroll
    for (int p = 0; p < PER; ++p) tile[tid + p * KN_THREADS] = make_key(rb, tid + p * KN_THREADS, N2);
    __syncthreads();

    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * KN_TILE;
      const float4 *tl = tile + (t & 1) * KN_TILE;
      const bool more = t + 1 < ntiles;
      float4 nxt[PER];
      if (more) {
#pragma unroll
        for (int p = 0; p < PER; ++p) nxt[p] = make_key(rb, t0 + KN_TILE + tid + p * KN_THREADS, N2);
      }

      // Drain every candidate buffer of this thread into its sorted lists (tile-local indices).
      auto drain = [&]() {
#pragma unroll
        for (int s = 0; s < Q; ++s) {
          float *d_s = ld + ((size_t)s * k) * KN_THREADS + tid;
          int *i_s = li + ((size_t)s * k) * KN_THREADS + tid;
          const int *b_s = buf + (s * KN_CAP) * KN_THREADS + tid;
          for (int c = 0; c < cnt[s]; ++c) {
            const int u = b_s[c * KN_THREADS];
            const int j = t0 + u;
            if (j >= N2) continue;
            const float4 r = tl[u];
            const float d = sqdist<float>(r.x, r.y, r.z, qx[s], qy[s], qz[s]);
            if (nk[s] == k && !(d < d_s[(k - 1) * KN_THREADS])) continue;
            int pos = nk[s] < k ? nk[s] : k - 1;
            while (pos > 0 && d < d_s[(pos - 1) * KN_THREADS]) {
              d_s[pos * KN_THREADS] = d_s[(pos - 1) * KN_THREADS];
              i_s[pos * KN_THREADS] = i_s[(pos - 1) * KN_THREADS];
              --pos;
            }
            d_s[pos * KN_THREADS] = d;
            i_s[pos * KN_THREADS] = j;
            if (nk[s] < k) ++nk[s];
          }
          cnt[s] = 0;
          if (nk[s] == k && thr[s] != -pinf())
            thr[s] = sweep_threshold(d_s[(k - 1) * KN_THREADS], sweep_qq(qx[s], qy[s], qz[s]));
        }
      };

      const int lim = (min(KN_TILE, N2 - t0) + KN_STEP - 1) & ~(KN_STEP - 1);
      for (int u0 = 0; u0 < lim; u0 += KN_STEP) {
        bool crowded = false;
#pragma unroll
        for (int s = 0; s < Q; ++s) crowded |= cnt[s] > KN_CAP - KN_STEP;
        if (__any_sync(0xffffffffu, crowded)) drain();
        // All filter values of the step first (independent FMA chains), then the appends.
        float a[KN_STEP][Q];
#pragma unroll
        for (int uu = 0; uu < KN_STEP; ++uu) {
          const float4 r = tl[u0 + uu];
#pragma unroll
          for (int s = 0; s < Q; ++s) a[uu][s] = sweep_lower(mx[s], my[s], mz[s], r);
        }
#pragma unroll
        for (int uu = 0; uu < KN_STEP; ++uu) {
#pragma unroll
          for (int s = 0; s < Q; ++s) {
            if (!(a[uu][s] >= thr[s])) {
              buf[(s * KN_CAP + cnt[s]) * KN_THREADS + tid] = u0 + uu;
              ++cnt[s];
            }
          }
        }
      }
      drain();  // candidates refer to this tile's buffer, which is about to be recycled

      if (more) {
        float4 *nx = tile + ((t + 1) & 1) * KN_TILE;
#pragma unroll
        for (int p = 0; p < PER; ++p) nx[tid + p * KN_THREADS] = nxt[p];
      }
      __syncthreads();
    }

#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = i0 + s * KN_THREADS;
      if (i < N1) {
        float *od = dist + (b * N1 + i) * k;
        int64_t *oi = index + (b * N1 + i) * k;
        const float *d_s = ld + ((size_t)s * k) * KN_THREADS + tid;
        const int *i_s = li + ((size_t)s * k) * KN_THREADS + tid;
        for (int c = 0; c < k; ++c) {
          od[c] = d_s[c * KN_THREADS];
          oi[c] = (int64_t)i_s[c * KN_THREADS];
        }
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
knn_generic_kernel(const T *__restrict__ query, const T *__restrict__ key, int64_t B, int64_t N1, int64_t N2,
                   int64_t k, T *__restrict__ dist, int64_t *__restrict__ index, int64_t blocks_total) {
  constexpr int TILE = 256;
  __shared__ T sx[TILE], sy[TILE], sz[TILE];
  const int tid = threadIdx.x;
  const int64_t chunks = (N1 + TILE - 1) / TILE;
  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int64_t i = (blk % chunks) * TILE + tid;
    const bool valid = i < N1;
    T qx = 0, qy = 0, qz = 0;
    if (valid) {
      const T *q = query + (b * N1 + i) * 3;
      qx = q[0];
      qy = q[1];
      qz = q[2];
    }
    T *od = dist + (b * N1 + (valid ? i : 0)) * k;
    int64_t *oi = index + (b * N1 + (valid ? i : 0)) * k;
    int64_t cnt = 0;
    T last = Exact<T>::inf();
    const T *rb = key + b * N2 * 3;
    for (int64_t t0 = 0; t0 < N2; t0 += TILE) {
      const int64_t jl = t0 + tid;
      if (jl < N2) {
        sx[tid] = rb[jl * 3 + 0];
        sy[tid] = rb[jl * 3 + 1];
        sz[tid] = rb[jl * 3 + 2];
      }
      __syncthreads();
      const int lim = (int)((N2 - t0) < TILE ? (N2 - t0) : TILE);
      if (valid) {
        for (int u = 0; u < lim; ++u) {
          const T d = sqdist<T>(sx[u], sy[u], sz[u], qx, qy, qz);
          if (cnt == k && !(d < last)) continue;
          int64_t pos = cnt < k ? cnt : k - 1;
          while (pos > 0 && d < od[pos - 1]) {
            od[pos] = od[pos - 1];
            oi[pos] = oi[pos - 1];
            --pos;
          }
          od[pos] = d;
          oi[pos] = t0 + u;
          if (cnt < k) ++cnt;
          if (cnt == k) last = od[k - 1];
        }
      }
      __syncthreads();
    }
  }
}

template <typename T>
int knn_generic(const T *query, const T *key, int64_t B, int64_t N1, int64_t N2, int64_t k, T *dist,
                int64_t *index, cudaStream_t st) {
  const int64_t total = B * ((N1 + 255) / 256);
  if (total == 0) return TK3D_OK;
  const int64_t cap = (int64_t)sm_count() * 64;
  knn_generic_kernel<T><<<(unsigned)(total < cap ? total : cap), 256, 0, st>>>(query, key, B, N1, N2, k, dist, index,
                                                                              total);
  return check_launch("knn_generic_kernel");
}

template <int K, int Q>
int knn_small(const float *query, const float *key, int64_t B, int N1, int N2, float *dist, int64_t *index,
              cudaStream_t st) {
  const int64_t per = KN_THREADS * Q;
  const int64_t total = B * ((N1 + per - 1) / per);
  const int64_t cap = (int64_t)sm_count() * 256;
  knn_small_kernel<K, Q><<<(unsigned)(total < cap ? total : cap), KN_THREADS, 0, st>>>(query, key, B, N1, N2, dist,
                                                                                      index, total);
  return check_launch("knn_small_kernel");
}

template <int K>
int knn_small_q(const float *query, const float *key, int64_t B, int N1, int N2, float *dist, int64_t *index,
                cudaStream_t st) {
  const int64_t sms = sm_count();
  if (B * (int64_t)N1 >= sms * 4 * KN_THREADS * 4) return knn_small<K, 4>(query, key, B, N1, N2, dist, index, st);
  if (B * (int64_t)N1 >= sms * 2 * KN_THREADS * 2) return knn_small<K, 2>(query, key, B, N1, N2, dist, index, st);
  return knn_small<K, 1>(query, key, B, N1, N2, dist, index, st);
}

size_t buffered_smem(int Q, int k) {
  return (size_t)2 * KN_TILE * 16 + (size_t)Q * k * KN_THREADS * 8 + (size_t)Q * KN_CAP * KN_THREADS * 4;
}

template <int Q>
int knn_buffered(const float *query, const float *key, int64_t B, int N1, int N2, int k, float *dist,
                 int64_t *index, cudaStream_t st) {
  const int64_t per = KN_THREADS * Q;
  const int64_t total = B * ((N1 + per - 1) / per);
  const size_t smem = buffered_smem(Q, k);
  TK3D_CUDA(cudaFuncSetAttribute(knn_buffered_kernel<Q>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int64_t cap = (int64_t)sm_count() * 64;
  knn_buffered_kernel<Q><<<(unsigned)(total < cap ? total : cap), KN_THREADS, smem, st>>>(query, key, B, N1, N2, k,
                                                                                        dist, index, total);
  return check_launch("knn_buffered_kernel");
}

}  // namespace
}  // namespace tk3d

using namespace tk3d;

extern "C" int tk3d_knn(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, int64_t k,
                        void *distance, int64_t *index, int dtype, void *stream) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "knn: dtype %d", dtype);
  TK3D_REQUIRE(B >= 0 && N1 >= 0 && N2 >= 0, TK3D_ERR_SHAPE, "knn: negative size");
  TK3D_REQUIRE(k >= 1, TK3D_ERR_K, "knn: k must be >= 1 (got %lld)", (long long)k);
  TK3D_REQUIRE(N2 >= k, TK3D_ERR_K, "knn: k=%lld exceeds the %lld key points", (long long)k, (long long)N2);
  TK3D_REQUIRE(N1 < (1LL << 30) && N2 < (1LL << 30), TK3D_ERR_SHAPE, "knn: clouds limited to 2^30 points");
  if (B * N1 == 0) return TK3D_OK;
  TK3D_REQUIRE(query && key && distance && index, TK3D_ERR_NULL, "knn: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F64)
    return knn_generic<double>((const double *)query, (const double *)key, B, N1, N2, k, (double *)distance, index,
                               st);
  const float *q = (const float *)query, *r = (const float *)key;
  float *d = (float *)distance;
  switch (k) {
    case 1: return knn_small_q<1>(q, r, B, (int)N1, (int)N2, d, index, st);
    case 2: return knn_small_q<2>(q, r, B, (int)N1, (int)N2, d, index, st);
    case 3: return knn_small_q<3>(q, r, B, (int)N1, (int)N2, d, index, st);
    case 4: return knn_small_q<4>(q, r, B, (int)N1, (int)N2, d, index, st);
    default: break;
  }
  if (k <= 128) {
    const int64_t sms = sm_count();
    if (k <= 32 && B * N1 >= sms * 2 * KN_THREADS * 2)
      return knn_buffered<2>(q, r, B, (int)N1, (int)N2, (int)k, d, index, st);
    return knn_buffered<1>(q, r, B, (int)N1, (int)N2, (int)k, d, index, st);
  }
  return knn_generic<float>(q, r, B, N1, N2, k, d, index, st);
}
