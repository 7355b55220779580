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

// Barrier of one 128-thread group of a larger block (named barrier 1 + group).
__device__ __forceinline__ void group_barrier(int grp) {
  asm volatile("bar.sync %0, 128;" ::"r"(grp + 1) : "memory");
}

// Verify path of one filter group (8 / Q keys starting at tile slot u0, global index t0 + u0):
// recompute the exact distance of every (key, query) pair whose filter value passed and update the
// running minimum in ascending key order with a strict "<".  With two queries per thread, m[s] is
// the smallest filter value of query s over the group, and a query none of whose values passes is
// skipped as a whole.  No bounds test: padding keys carry a filter value of +inf, which no
// threshold admits.
template <int Q>
__device__ __forceinline__ void chamfer_verify(const float4 *tl, int u0, int t0, const float2 (&a)[4],
                                               const float (&m)[2], const float (&qx)[Q], const float (&qy)[Q],
                                               const float (&qz)[Q], float (&thr)[Q], float (&best)[Q],
                                               int (&arg)[Q]) {
  constexpr int GK = 8 / Q;
#pragma unroll
  for (int s = 0; s < Q; ++s) {
    if (Q != 2 || !(m[s] >= thr[s])) {
#pragma unroll
      for (int k = 0; k < GK; ++k) {
        const float av = (k & 1) ? a[(k >> 1) * Q + s].y : a[(k >> 1) * Q + s].x;
        if (!(av >= thr[s])) {
          const float4 r = sweep_load_key(tl, u0 + k);
          const float d = sqdist<float>(r.x, r.y, r.z, qx[s], qy[s], qz[s]);
          if (d < best[s]) {
            best[s] = d;
            arg[s] = t0 + u0 + k;
            thr[s] = sweep_threshold(d, sweep_qq(qx[s], qy[s], qz[s]));
          }
        }
      }
    }
  }
}

// LANES > 1: several lanes per query, for launches that cannot fill the GPU with one lane per query
// (their time is the critical path of a single warp).  The LANES lanes l, l + 32/LANES, ... of a
// warp hold the same Q queries and sweep every LANES-th key group of each tile; once per tile they
// exchange the smallest of their best distances -- any lane's best bounds the query's nearest
// distance; taken one ulp higher, because a key AT that distance with a lower index must still pass
// this lane's filter -- and at the end the best (distance, index) of all lanes is kept.  Same pairs
// per shared-memory load, LANES times the warps.
template <int Q, int MINB = 1, int UNR = 2, int CF_THREADS = 128, int LANES = 1>
__global__ void __launch_bounds__(CF_THREADS, MINB)
chamfer_fwd_fast_kernel(const float *__restrict__ xyz1, const float *__restrict__ xyz2, int64_t B, int N1, int N2,
                        float *__restrict__ dist1, int64_t *__restrict__ idx1, float *__restrict__ dist2,
                        int64_t *__restrict__ idx2, double *__restrict__ sums, int64_t blocks1,
                        int64_t blocks_total, XyzLayout l1, XyzLayout l2) {
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
    const XyzLayout lq = dir ? l2 : l1, lr = dir ? l1 : l2;
    constexpr int QL = 32 / LANES;                 // distinct queries (per s) in a warp
    constexpr int QPB = CF_THREADS * Q / LANES;    // queries per block
    const int chunks = (nq + QPB - 1) / QPB;
    const int64_t b = id / chunks;
    const int i0 = (int)(id % chunks) * QPB;
    const int part = (tid & 31) / QL;              // which of a query's LANES lanes this is
    auto qindex = [&](int s) {
      if (LANES > 1) return i0 + (tid >> 5) * (QL * Q) + s * QL + (tid & (QL - 1));
      return i0 + tid + s * CF_THREADS;
    };

    float qx[Q], qy[Q], qz[Q], thr[Q], best[Q];
    float pthr[Q];  // LANES > 1: threshold from the lanes' best distances at the last exchange
    float2 mx[Q], my[Q], mz[Q];
    int arg[Q];
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = qindex(s);
      pthr[s] = pinf;
      best[s] = pinf;
      arg[s] = -1;
      if (i < nq) {
        load_xyz(qpts + b * 3 * (int64_t)nq, i, lq, qx[s], qy[s], qz[s]);
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
          float x, y, z;
          load_xyz(rb, u, lr, x, y, z);
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
            load_xyz(rb, j, lr, px[p], py[p], pz[p]);
          } else {
            px[p] = py[p] = pz[p] = 0.f;
          }
        }
      }

      constexpr int STEP = LANES * GK;  // the lanes of a query take every LANES-th group
      const int lim = (cnt + STEP - 1) / STEP * STEP;
#pragma unroll UNR
      for (int u0 = part * GK; u0 < lim; u0 += STEP) {
        float2 a[4];
        float m[2];
        bool any;
        if constexpr (Q == 2) any = sweep_group2_gated(tl + u0, mx, my, mz, thr, a, m);
        else any = sweep_group2<Q, true>(tl + u0, mx, my, mz, thr, a);
        if (__builtin_expect(any, 0)) {
          chamfer_verify<Q>(tl, u0, t0, a, m, qx, qy, qz, thr, best, arg);
          if constexpr (LANES > 1) {
#pragma unroll
            for (int s = 0; s < Q; ++s) thr[s] = fminf(thr[s], pthr[s]);
          }
        }
      }
      if constexpr (LANES > 1) {
#pragma unroll
        for (int s = 0; s < Q; ++s) {
          float pk = best[s];  // smallest best distance among the query's lanes (a NaN is never smaller)
#pragma unroll
          for (int o = QL; o < 32; o <<= 1) pk = fminf(pk, __shfl_xor_sync(0xffffffffu, pk, o));
          const float up = pk < pinf ? __uint_as_float(__float_as_uint(pk) + 1u) : pk;  // pk >= +0
          pthr[s] = sweep_threshold(up, sweep_qq(qx[s], qy[s], qz[s]));
          thr[s] = fminf(thr[s], pthr[s]);
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

    if constexpr (LANES > 1) {  // the best (distance, index) over the lanes, in butterfly steps
#pragma unroll
      for (int o = QL; o < 32; o <<= 1) {
#pragma unroll
        for (int s = 0; s < Q; ++s) {
          const float od = __shfl_xor_sync(0xffffffffu, best[s], o);
          const int oi = __shfl_xor_sync(0xffffffffu, arg[s], o);
          if (oi >= 0 && (arg[s] < 0 || od < best[s] || (od == best[s] && oi < arg[s]))) {
            best[s] = od;
            arg[s] = oi;
          }
        }
      }
    }
    float *dist = dir ? dist2 : dist1;
    int64_t *idx = dir ? idx2 : idx1;
    double psum = 0.0;
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = qindex(s);
      if (i < nq && part == 0) {
        dist[b * nq + i] = best[s];
        idx[b * nq + i] = (int64_t)arg[s];
        psum += (double)best[s];
      }
    }
    if (sums != nullptr) {
      psum = warp_sum(psum);
      if ((tid & 31) == 0) ssum[tid >> 5] = psum;
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

template <int Q, int MINB = 1, int UNR = 2, int CF_THREADS = 128, int LANES = 1>
int launch(const float *xyz1, const float *xyz2, int64_t B, int N1, int N2, float *dist1, int64_t *idx1,
           float *dist2, int64_t *idx2, double *sums, cudaStream_t st, XyzLayout l1, XyzLayout l2, int only_dir = -1) {
  // only_dir: -1 = both directions in this launch, 0 = cloud 1 -> cloud 2 only, 1 = the other one
  const int64_t per = CF_THREADS * Q / LANES;
  const int64_t blocks1 = only_dir == 1 ? 0 : B * ((N1 + per - 1) / per);
  const int64_t blocks2 = only_dir == 0 ? 0 : B * ((N2 + per - 1) / per);
  const int64_t total = blocks1 + blocks2;
  if (total == 0) return TK3D_OK;
  const int64_t cap = (int64_t)sm_count() * 256;
  const unsigned grid = (unsigned)(total < cap ? total : cap);
  chamfer_fwd_fast_kernel<Q, MINB, UNR, CF_THREADS, LANES><<<grid, CF_THREADS, 0, st>>>(
      xyz1, xyz2, B, N1, N2, dist1, idx1, dist2, idx2, sums, blocks1, total, l1, l2);
  return check_launch("chamfer_fwd_fast_kernel");
}

// ---- one block per SM, for launches of one or two rounds of tasks --------------------------------
// A launch of the kernel above pays a fixed cost of about 15 % of the time one round of tasks
// takes (measured for task lengths from 4096 to 32768 keys), which is nothing for many rounds
// but all of it for one rank's share of a batch split over several GPUs (8 clouds of 16384
// points are 1024 tasks for 148 SMs: 0.80 ms where 0.70 ms would be an eighth of the 64-cloud
// launch).  Measured on B200, the same sweep run as ONE block of 896 threads per SM -- seven
// groups of 128 threads, each group working through its own task with its own pair of tile
// buffers and its own named barrier, exactly like a block of the kernel above -- does not pay it
// (0.74 ms), while over many rounds it is about 5 % slower than independently scheduled blocks
// (its groups are bound to their block, so an SM's last tasks of a round run with the SM partly
// empty).  The launcher therefore picks this kernel only for one or two nearly full rounds of
// tasks.  896 threads leave 72 registers per thread.
template <int UNR>
__global__ void __launch_bounds__(896, 1)
chamfer_fwd_smwide_kernel(const float *__restrict__ xyz1, const float *__restrict__ xyz2, int N1, int N2,
                          float *__restrict__ dist1, int64_t *__restrict__ idx1, float *__restrict__ dist2,
                          int64_t *__restrict__ idx2, double *__restrict__ sums, int blocks1,
                          int blocks_total, XyzLayout l1, XyzLayout l2) {
  constexpr int Q = 2, TH = 128;
  constexpr int PER = CF_TILE / TH;
  extern __shared__ float4 group_tiles[];  // [groups][2][CF_TILE]
  const int tid = threadIdx.x & (TH - 1);
  const int grp = threadIdx.x >> 7;
  const int groups = blockDim.x >> 7;
  float4(*tile)[CF_TILE] = reinterpret_cast<float4(*)[CF_TILE]>(group_tiles + (size_t)grp * 2 * CF_TILE);
  const float pinf = __int_as_float(0x7f800000);

  // Every group walks its own tasks; groups never wait for one another.
  for (int blk = blockIdx.x * groups + grp; blk < blocks_total; blk += gridDim.x * groups) {
    const int dir = blk >= blocks1;
    const int id = dir ? blk - blocks1 : blk;
    const float *qpts = dir ? xyz2 : xyz1;
    const float *rpts = dir ? xyz1 : xyz2;
    const int nq = dir ? N2 : N1;
    const int nr = dir ? N1 : N2;
    const XyzLayout lq = dir ? l2 : l1, lr = dir ? l1 : l2;
    const int chunks = (nq + TH * Q - 1) / (TH * Q);
    const int64_t b = id / chunks;
    const int i0 = (id % chunks) * (TH * Q) + tid;

    float qx[Q], qy[Q], qz[Q], thr[Q], best[Q];
    float2 mx[Q], my[Q], mz[Q];
    int arg[Q];
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = i0 + s * TH;
      best[s] = pinf;
      arg[s] = -1;
      if (i < nq) {
        load_xyz(qpts + b * 3 * (int64_t)nq, i, lq, qx[s], qy[s], qz[s]);
        thr[s] = pinf;  // accept everything until a first candidate is verified
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
    if (ntiles > 0) {
#pragma unroll
      for (int p = 0; p < PER; ++p) {
        const int u = tid + p * TH;
        if (u < nr) {
          float x, y, z;
          load_xyz(rb, u, lr, x, y, z);
          sweep_store_key(tile[0], u, x, y, z, sweep_key_w(x, y, z));
        } else {
          sweep_store_key(tile[0], u, 0.f, 0.f, 0.f, pinf);
        }
      }
    }
    group_barrier(grp);

    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * CF_TILE;
      const int cnt = min(CF_TILE, nr - t0);
      const float4 *tl = tile[t & 1];

      float px[PER], py[PER], pz[PER];
      const bool more = t + 1 < ntiles;
      if (more) {
#pragma unroll
        for (int p = 0; p < PER; ++p) {
          const int j = t0 + CF_TILE + tid + p * TH;
          if (j < nr) {
            load_xyz(rb, j, lr, px[p], py[p], pz[p]);
          } else {
            px[p] = py[p] = pz[p] = 0.f;
          }
        }
      }

      const int lim = (cnt + 3) / 4 * 4;
#pragma unroll UNR
      for (int u0 = 0; u0 < lim; u0 += 4) {
        float2 a[4];
        float m[2];
        if (__builtin_expect(sweep_group2_gated(tl + u0, mx, my, mz, thr, a, m), 0))
          chamfer_verify<Q>(tl, u0, t0, a, m, qx, qy, qz, thr, best, arg);
      }

      if (more) {
        float4 *nx = tile[(t + 1) & 1];
#pragma unroll
        for (int p = 0; p < PER; ++p) {
          const int u = tid + p * TH;
          if (t0 + CF_TILE + u < nr)
            sweep_store_key(nx, u, px[p], py[p], pz[p], sweep_key_w(px[p], py[p], pz[p]));
          else
            sweep_store_key(nx, u, 0.f, 0.f, 0.f, pinf);
        }
      }
      group_barrier(grp);
    }

    float *dist = dir ? dist2 : dist1;
    int64_t *idx = dir ? idx2 : idx1;
    double part = 0.0;
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = i0 + s * TH;
      if (i < nq) {
        dist[b * nq + i] = best[s];
        idx[b * nq + i] = (int64_t)arg[s];
        part += (double)best[s];
      }
    }
    if (sums != nullptr) {
      part = warp_sum(part);
      if ((tid & 31) == 0) atomicAdd(sums + dir, part);
    }
  }
}

constexpr int SMWIDE_GROUPS = 7;

int launch_smwide(const float *xyz1, const float *xyz2, int64_t B, int N1, int N2, float *dist1, int64_t *idx1,
                  float *dist2, int64_t *idx2, double *sums, cudaStream_t st, XyzLayout l1, XyzLayout l2) {
  const int64_t blocks1 = B * ((N1 + 255) / 256), blocks2 = B * ((N2 + 255) / 256);
  const int64_t total = blocks1 + blocks2;
  const size_t smem = (size_t)SMWIDE_GROUPS * 2 * CF_TILE * sizeof(float4);  // 112 KB
  TK3D_CUDA(raise_smem_limit((const void *)chamfer_fwd_smwide_kernel<4>, (int)smem));
  const int64_t blocks = (total + SMWIDE_GROUPS - 1) / SMWIDE_GROUPS;
  const int64_t cap = sm_count();
  chamfer_fwd_smwide_kernel<4><<<(unsigned)(blocks < cap ? blocks : cap), 128 * SMWIDE_GROUPS, smem, st>>>(
      xyz1, xyz2, N1, N2, dist1, idx1, dist2, idx2, sums, (int)blocks1, (int)total, l1, l2);
  return check_launch("chamfer_fwd_smwide_kernel");
}

}  // namespace

// 0: one query per thread, 1: one block per SM, 2: two queries per thread in independent blocks.
static int chamfer_fwd_f32_plan(int64_t B, int64_t N1, int64_t N2) {
  const int64_t queries = B * (N1 + N2);
  const int64_t sms = sm_count();
  // Queries per thread: more register tiling when there is enough work to fill the GPU with it.
  if (queries < sms * 2 * 128 * 2) return 0;
  const int64_t tasks = B * ((N1 + 255) / 256) + B * ((N2 + 255) / 256);
  // In units of one round (seven tasks per SM): independent blocks take about rounds + 0.15, the
  // one-block-per-SM kernel 1.055 x the rounds rounded up.
  const int64_t round = SMWIDE_GROUPS * sms, rounds_up = (tasks + round - 1) / round;
  if (tasks < (1LL << 30) && 1055 * rounds_up * round < 1000 * tasks + 150 * round) return 1;
  return 2;
}

const char *chamfer_fwd_f32_kernel_name(int64_t B, int64_t N1, int64_t N2) {
  static const char *const names[3] = {"chamfer_fwd_fast_kernel<1>", "chamfer_fwd_smwide_kernel",
                                       "chamfer_fwd_fast_kernel<2>"};
  return names[chamfer_fwd_f32_plan(B, N1, N2)];
}

// Lanes per query for launches with one query per thread; `nq` counts the queries of both
// directions of a symmetric problem.  Measured on B200 (148 SMs), forward of both directions, ms:
//   queries  1 lane   2 lanes  4 lanes  8 lanes    (clouds)
//   65536    0.062    0.076    0.106    0.177      16 x 2048 x 2048
//   32768    0.082    0.064    0.098    0.171      4 x 4096 x 4096
//   24096    0.141    0.091    0.075    0.107      2 x 2048 x 10000
//   16384    0.035    0.027    0.025    0.034      8 x 1024 x 1024
//    4096    0.034    0.024    0.024    0.024      2 x 1024 x 1024
static int chamfer_lanes(int64_t nq) {
  const int64_t sms = sm_count();
  if (nq * 3 > sms * 1000) return 1;   // above about 49 000 queries on 148 SMs
  if (nq * 6 > sms * 1000) return 2;   // above about 24 600
  if (nq * 48 > sms * 1000) return 4;  // above about 3 000
  return 8;
}

// One direction (or both) with one query per thread and the lane count that suits `nq` queries.
static int launch_lanes(int64_t nq, const float *xyz1, const float *xyz2, int64_t B, int N1, int N2, float *dist1,
                        int64_t *idx1, float *dist2, int64_t *idx2, double *sums, cudaStream_t st, XyzLayout l1,
                        XyzLayout l2, int only_dir) {
  switch (chamfer_lanes(nq)) {
    case 8: return launch<1, 1, 2, 128, 8>(xyz1, xyz2, B, N1, N2, dist1, idx1, dist2, idx2, sums, st, l1, l2, only_dir);
    case 4: return launch<1, 1, 2, 128, 4>(xyz1, xyz2, B, N1, N2, dist1, idx1, dist2, idx2, sums, st, l1, l2, only_dir);
    case 2: return launch<1, 1, 2, 128, 2>(xyz1, xyz2, B, N1, N2, dist1, idx1, dist2, idx2, sums, st, l1, l2, only_dir);
    default: return launch<1, 1, 2>(xyz1, xyz2, B, N1, N2, dist1, idx1, dist2, idx2, sums, st, l1, l2, only_dir);
  }
}

int chamfer_fwd_f32_fast(const float *xyz1, const float *xyz2, int64_t B, int64_t N1, int64_t N2, float *dist1,
                         int64_t *idx1, float *dist2, int64_t *idx2, double *sums, cudaStream_t st, XyzLayout l1,
                         XyzLayout l2) {
  const int64_t sms = sm_count();
  const int64_t small = B * (N1 < N2 ? N1 : N2), large = B * (N1 < N2 ? N2 : N1);
  // Clouds of very different sizes: the direction with few queries sweeps the large cloud and is
  // the critical path, the other one is many queries against few keys.  Each gets its own launch
  // and its own shape (1 x 300 x 50000: 0.54 -> 0.19 ms).
  if (small > 0 && large >= 4 * small && 2 * small < sms * 2 * 128 * 2) {
    const int few = N1 < N2 ? 0 : 1;  // the direction whose queries are the small cloud
    int rc = launch_lanes(2 * small, xyz1, xyz2, B, (int)N1, (int)N2, dist1, idx1, dist2, idx2, sums, st, l1, l2, few);
    if (rc) return rc;
    if (2 * large < sms * 2 * 128 * 2)
      return launch_lanes(2 * large, xyz1, xyz2, B, (int)N1, (int)N2, dist1, idx1, dist2, idx2, sums, st, l1, l2,
                          1 - few);
    return launch<2, 6, 4>(xyz1, xyz2, B, (int)N1, (int)N2, dist1, idx1, dist2, idx2, sums, st, l1, l2, 1 - few);
  }
  // Measured on B200 (B=64, N=M=16384): two queries per thread, six resident blocks per SM and a
  // four-fold unrolled key loop beat four queries per thread by about 10 %.
  switch (chamfer_fwd_f32_plan(B, N1, N2)) {
    case 0:
      return launch_lanes(B * (N1 + N2), xyz1, xyz2, B, (int)N1, (int)N2, dist1, idx1, dist2, idx2, sums, st, l1, l2, -1);
    case 1: return launch_smwide(xyz1, xyz2, B, (int)N1, (int)N2, dist1, idx1, dist2, idx2, sums, st, l1, l2);
    default: return launch<2, 6, 4>(xyz1, xyz2, B, (int)N1, (int)N2, dist1, idx1, dist2, idx2, sums, st, l1, l2);
  }
}

}  // namespace tk3d

TK3D_BOUNDS_TU(chamfer_fast)
