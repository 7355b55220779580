// Chamfer forward, fp32 fast path: register-tiled filter-then-verify sweep (see sweep.cuh).
//
// A block of 128 threads owns 128*Q query points (Q = 2 per thread, 128 apart so loads and stores
// coalesce) of one cloud and sweeps the whole partner cloud in 512-point tiles.  A tile is staged
// in shared memory in the pair layout of sweep.cuh, (x0,x1,y0,y1)(z0,z1,w0,w1) per two keys; every
// lane reads the same 32 bytes (two broadcast LDS.128 per key pair) and one packed FMA evaluates
// the filter of one query against both keys.  The next tile's coordinates are fetched into
// registers before the current tile is processed and written to the other buffer afterwards, so
// global latency hides behind the arithmetic with a single barrier per tile.
//
// Per (key, query) pair the hot loop issues 1.5 packed FMA, half a three-input minimum and a
// quarter of a compare (eight pairs share two compares and one branch); the exactly rounded
// distance is recomputed only for pairs that pass the filter (about ln(M) + a few per query), and
// the running minimum is updated with a strict "<" in ascending key order, so the lowest index
// wins ties.
//
// Both directions run in one launch; each block adds its partial sum of distances to `sums`.
#include "sweep.cuh"

namespace tk3d {

namespace {

constexpr int CF_TILE = 512;

template <int Q, int MINB = 1, int UNR = 2, int CF_THREADS = 128>
__global__ void __launch_bounds__(CF_THREADS, MINB)
chamfer_fwd_fast_kernel(const float *__restrict__ xyz1, const float *__restrict__ xyz2, int64_t B, int N1, int N2,
                        float *__restrict__ dist1, int64_t *__restrict__ idx1, float *__restrict__ dist2,
                        int64_t *__restrict__ idx2, double *__restrict__ sums, int64_t blocks1,
                        int64_t blocks_total) {
  constexpr int PER = CF_TILE / CF_THREADS;
  constexpr int GK = 8 / Q;  // keys per filter group: eight (key, query) pairs share one branch
  __shared__ float4 tile[2][CF_TILE];
  __shared__ double ssum[CF_THREADS / 32];
  static_assert(CF_TILE % CF_THREADS == 0, "tile is staged in whole rounds of the block");
  const int tid = threadIdx.x;
  const float pinf = __int_as_float(0x7f800000);

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int dir = blk >= blocks1;
    const int64_t id = dir ? blk - blocks1 : blk;
    const float *qpts = dir ? xyz2 : xyz1;
    const float *rpts = dir ? xyz1 : xyz2;
    const int nq = dir ? N2 : N1;
    const int nr = dir ? N1 : N2;
    const int chunks = (nq + CF_THREADS * Q - 1) / (CF_THREADS * Q);
    const int64_t b = id / chunks;
    const int i0 = (int)(id % chunks) * (CF_THREADS * Q) + tid;

    float qx[Q], qy[Q], qz[Q], thr[Q], best[Q];
    float2 mx[Q], my[Q], mz[Q];
    int arg[Q];
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = i0 + s * CF_THREADS;
      best[s] = pinf;
      arg[s] = -1;
      if (i < nq) {
        const float *q = qpts + (b * nq + i) * 3;
        qx[s] = q[0];
        qy[s] = q[1];
        qz[s] = q[2];
        thr[s] = pinf;  // accept everything until a first candidate is verified (minima-based test)
      } else {
        qx[s] = qy[s] = qz[s] = 0.f;
        thr[s] = -pinf;  // never passes
      }
      mx[s] = make_float2(-2.f * qx[s], -2.f * qx[s]);
      my[s] = make_float2(-2.f * qy[s], -2.f * qy[s]);
      mz[s] = make_float2(-2.f * qz[s], -2.f * qz[s]);
    }

    const float *rb = rpts + b * (int64_t)nr * 3;
    const int ntiles = (nr + CF_TILE - 1) / CF_TILE;

    // Prologue: stage tile 0 (padded to the full tile with points that cannot be accepted).
    if (ntiles > 0) {
#pragma unroll
      for (int p = 0; p < PER; ++p) {
        const int u = tid + p * CF_THREADS;
        if (u < nr) {
          const float x = rb[u * 3 + 0], y = rb[u * 3 + 1], z = rb[u * 3 + 2];
          sweep_store_key(tile[0], u, x, y, z, sweep_key_w(x, y, z));
        } else {
          sweep_store_key(tile[0], u, 0.f, 0.f, 0.f, pinf);
        }
      }
    }
    __syncthreads();

    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * CF_TILE;
      const int cnt = min(CF_TILE, nr - t0);
      const float4 *tl = tile[t & 1];

      // Fetch the next tile's coordinates into registers.
      float px[PER], py[PER], pz[PER];
      const bool more = t + 1 < ntiles;
      if (more) {
#pragma unroll
        for (int p = 0; p < PER; ++p) {
          const int j = t0 + CF_TILE + tid + p * CF_THREADS;
          if (j < nr) {
            px[p] = rb[(int64_t)j * 3 + 0];
            py[p] = rb[(int64_t)j * 3 + 1];
            pz[p] = rb[(int64_t)j * 3 + 2];
          } else {
            px[p] = py[p] = pz[p] = 0.f;
          }
        }
      }

      const int lim = (cnt + GK - 1) / GK * GK;
#pragma unroll UNR
      for (int u0 = 0; u0 < lim; u0 += GK) {
        float2 a[4];
        if (__builtin_expect(sweep_group2<Q, true>(tl + u0, mx, my, mz, thr, a), 0)) {
#pragma unroll
          for (int p = 0; p < GK / 2; ++p) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // no bounds test: padding keys carry a filter value of +inf, which no threshold admits
              const int j = t0 + u0 + 2 * p + h;
              const float4 r = sweep_load_key(tl, u0 + 2 * p + h);
#pragma unroll
              for (int s = 0; s < Q; ++s) {
                const float av = h ? a[p * Q + s].y : a[p * Q + s].x;
                if (!(av >= thr[s])) {
                  const float d = sqdist<float>(r.x, r.y, r.z, qx[s], qy[s], qz[s]);
                  if (d < best[s]) {
                    best[s] = d;
                    arg[s] = j;
                    thr[s] = sweep_threshold(d, sweep_qq(qx[s], qy[s], qz[s]));
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
        for (int p = 0; p < PER; ++p) {
          const int u = tid + p * CF_THREADS;
          if (t0 + CF_TILE + u < nr)
            sweep_store_key(nx, u, px[p], py[p], pz[p], sweep_key_w(px[p], py[p], pz[p]));
          else
            sweep_store_key(nx, u, 0.f, 0.f, 0.f, pinf);
        }
      }
      __syncthreads();
    }

    float *dist = dir ? dist2 : dist1;
    int64_t *idx = dir ? idx2 : idx1;
    double part = 0.0;
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = i0 + s * CF_THREADS;
      if (i < nq) {
        dist[b * nq + i] = best[s];
        idx[b * nq + i] = (int64_t)arg[s];
        part += (double)best[s];
      }
    }
    if (sums != nullptr) {
      part = warp_sum(part);
      if ((tid & 31) == 0) ssum[tid >> 5] = part;
      __syncthreads();
      if (tid == 0) {
        double tot = 0;
#pragma unroll
        for (int w = 0; w < CF_THREADS / 32; ++w) tot += ssum[w];
        atomicAdd(sums + dir, tot);
      }
    }
    __syncthreads();
  }
}

template <int Q, int MINB = 1, int UNR = 2, int CF_THREADS = 128>
int launch(const float *xyz1, const float *xyz2, int64_t B, int N1, int N2, float *dist1, int64_t *idx1,
           float *dist2, int64_t *idx2, double *sums, cudaStream_t st) {
  const int64_t per = CF_THREADS * Q;
  const int64_t blocks1 = B * ((N1 + per - 1) / per), blocks2 = B * ((N2 + per - 1) / per);
  const int64_t total = blocks1 + blocks2;
  if (total == 0) return TK3D_OK;
  const int64_t cap = (int64_t)sm_count() * 256;
  const unsigned grid = (unsigned)(total < cap ? total : cap);
  chamfer_fwd_fast_kernel<Q, MINB, UNR, CF_THREADS><<<grid, CF_THREADS, 0, st>>>(xyz1, xyz2, B, N1, N2, dist1, idx1, dist2, idx2, sums,
                                                           blocks1, total);
  return check_launch("chamfer_fwd_fast_kernel");
}

}  // namespace

int chamfer_fwd_f32_fast(const float *xyz1, const float *xyz2, int64_t B, int64_t N1, int64_t N2, float *dist1,
                         int64_t *idx1, float *dist2, int64_t *idx2, double *sums, cudaStream_t st) {
  // Queries per thread: more register tiling when there is enough work to fill the GPU with it.
  const int64_t queries = B * (N1 + N2);
  const int64_t sms = sm_count();
  constexpr int CF_THREADS = 128;
  // Measured on B200 (B=64, N=M=16384): two queries per thread, six resident blocks per SM and a
  // four-fold unrolled key loop beat four queries per thread by about 10 %.
  if (queries >= sms * 2 * CF_THREADS * 2)
    return launch<2, 6, 4>(xyz1, xyz2, B, (int)N1, (int)N2, dist1, idx1, dist2, idx2, sums, st);
  return launch<1, 1, 2>(xyz1, xyz2, B, (int)N1, (int)N2, dist1, idx1, dist2, idx2, sums, st);
}

}  // namespace tk3d
