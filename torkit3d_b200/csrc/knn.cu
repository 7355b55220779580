// Brute-force k nearest neighbours (squared distances, rows sorted ascending by (distance, index)).
//
// Four kernels here, two more in files of their own (knn_select.cu: float32 with 64 < k <= 256, or
// 40 < k with fewer than 16 keys per wanted neighbour, by radix selection; knn_split.cu: float64
// with few queries):
//   knn_small_kernel<K,Q>  fp32, k <= 4: per-thread top-K in registers, filter-then-verify sweep
//                          (sweep.cuh), insertion straight from the verify branch.  With k << N2
//                          the branch is rare (about k ln(N2/k) times per query).
//   knn_twopass_kernel     fp32, 4 < k <= 64 (and N2 >= 4 k, at least 256): pass 1 bounds the k-th distance from
//                          class minima of the filter value, pass 2 collects the few candidates
//                          below the bound, exact selection among them (see the kernel's header).
//   knn_buffered_kernel<Q> fp32, other k <= 40 (small key clouds): same filter, but passing keys are only appended
//                          (predicated store, no branch) to a small per-query candidate buffer in
//                          shared memory; buffers are drained into per-query sorted lists (also in
//                          shared memory) by the whole warp at once, when any lane's buffer is
//                          nearly full and at the end of every key tile.  This keeps the lanes of a
//                          warp in step even when k ln(N2/k) is not small against N2.
//   knn_generic_kernel<T>  any type / any k: one query per thread, exact distances, sorted list kept
//                          directly in the output rows.
// All of them take decisions on the exactly rounded distance and scan keys in ascending order with
// strict comparisons, so the retained set and its order are reproducible bit for bit.
#include <stdlib.h>

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
__device__ __forceinline__ float4 make_key(const float *__restrict__ rb, int j, int nr, XyzLayout l) {
  if (j < nr) {
    float x, y, z;
    load_xyz(rb, j, l, x, y, z);
    return make_float4(x, y, z, sweep_key_w(x, y, z));
  }
  return make_float4(0.f, 0.f, 0.f, pinf());
}

// LANES > 1: several lanes per query.  The LANES lanes l, l + 32/LANES, ... of a warp hold the same
// Q queries and sweep every LANES-th key group of each tile, each into its own sorted list; once
// per tile they exchange their lists' distances and continue with the k-th smallest of the union
// as the bound (the lists hold disjoint keys, so that bounds the query's k-th distance), and at the
// end the lists are merged by (distance, index) in log2(LANES) butterfly steps.  Same pairs per shared-memory load, same staging, but
// LANES times the warps for a given number of queries: for launches that cannot fill the GPU with
// one lane per query, whose time is the critical path of a single warp.
template <int K, int Q, int LANES = 1, bool FIRSTX = false>
__global__ void __launch_bounds__(KN_THREADS)
knn_small_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2,
                 float *__restrict__ dist, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  constexpr int TILE = 512, PER = TILE / KN_THREADS;
  constexpr int GK = 8 / Q;  // keys per filter group: eight (key, query) pairs share one branch
  __shared__ float4 tile[2][TILE];  // pair layout of sweep.cuh
  const int tid = threadIdx.x;
  constexpr bool HALF = LANES > 1;
  constexpr int QL = 32 / LANES;                      // distinct queries (per s) in a warp
  constexpr int QPB = KN_THREADS * Q / LANES;         // queries per block
  const int chunks = (N1 + QPB - 1) / QPB;
  const int half = (tid & 31) / QL;                   // which of a query's LANES lanes this is

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int i0 = (int)(blk % chunks) * QPB;
    // query s of this thread
    auto qindex = [&](int s) {
      if (HALF) return i0 + (tid >> 5) * (QL * Q) + s * QL + (tid & (QL - 1));
      return i0 + tid + s * KN_THREADS;
    };
    float qx[Q], qy[Q], qz[Q], thr[Q];
    float pthr[Q];  // LANES > 1: threshold from the other lanes' k-th distances at the last exchange
    float2 mx[Q], my[Q], mz[Q];
    float kd[Q][K];
    int ki[Q][K];
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      pthr[s] = pinf();
      const int i = qindex(s);
      if (i < N1) {
        load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx[s], qy[s], qz[s]);
        thr[s] = pinf();  // accept everything until the list is full
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
      const float4 v = make_key(rb, u, N2, kl);
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
        for (int p = 0; p < PER; ++p) nxt[p] = make_key(rb, t0 + TILE + tid + p * KN_THREADS, N2, kl);
      }
      constexpr int STEP = LANES * GK;  // the lanes of a query take every LANES-th group
      const int lim = (min(TILE, N2 - t0) + STEP - 1) / STEP * STEP;
      // LANES > 1: another lane's k-th entry bounds this query's k-th entry too.  A key of this
      // lane's groups AT that distance may still precede it by index, so the bound is taken one
      // ulp above it: the filter guarantees a pass for d < bound only.  Once per tile: exchanging
      // four times per tile measured 20 % slower (it breaks up the unrolled loop).
      auto exchange = [&]() {
#pragma unroll
        for (int s = 0; s < Q; ++s) {
          // k-th smallest distance of the UNION of the lanes' lists (they hold disjoint keys): the
          // k smallest of two ascending lists a, b are min(a[c], b[K-1-c]), c = 0..K-1
          float e[K];
#pragma unroll
          for (int c = 0; c < K; ++c) e[c] = kd[s][c];
#pragma unroll
          for (int o = QL; o < 32; o <<= 1) {
            float pe[K];
#pragma unroll
            for (int c = 0; c < K; ++c) pe[c] = __shfl_xor_sync(0xffffffffu, e[c], o);
#pragma unroll
            for (int c = 0; c < K; ++c) e[c] = fminf(e[c], pe[K - 1 - c]);
            if (2 * o < 32) {  // another step follows: it needs the list in ascending order again
#pragma unroll
              for (int a_ = 0; a_ < K - 1; ++a_) {
#pragma unroll
                for (int c = 0; c < K - 1 - a_; ++c) {
                  const float lo = fminf(e[c], e[c + 1]), hi = fmaxf(e[c], e[c + 1]);
                  e[c] = lo;
                  e[c + 1] = hi;
                }
              }
            }
          }
          float pk = e[0];
#pragma unroll
          for (int c = 1; c < K; ++c) pk = fmaxf(pk, e[c]);
          const float up = pk < pinf() ? __uint_as_float(__float_as_uint(pk) + 1u) : pk;  // pk >= +0 or NaN
          pthr[s] = pk == pk ? sweep_threshold(up, sweep_qq(qx[s], qy[s], qz[s])) : pinf();
          thr[s] = fminf(thr[s], pthr[s]);
        }
      };
      auto sweep = [&](int ubeg, int uend) {
#pragma unroll 4
      for (int u0 = ubeg + half * GK; u0 < uend; u0 += STEP) {
        float2 a[4];
        float m[2];
        bool any;
        if constexpr (Q == 2) any = sweep_group2_gated(tl + u0, mx, my, mz, thr, a, m);
        else any = sweep_group2<Q, true>(tl + u0, mx, my, mz, thr, a);
        if (__builtin_expect(any, 0)) {
#pragma unroll
          for (int s = 0; s < Q; ++s) {
            // with two queries per thread, skip the one whose four filter values all fail
            if (Q != 2 || !(m[s] >= thr[s])) {
#pragma unroll
              for (int k = 0; k < GK; ++k) {
                // no bounds test: padding keys carry a filter value of +inf, which no threshold admits
                const float av = (k & 1) ? a[(k >> 1) * Q + s].y : a[(k >> 1) * Q + s].x;
                if (!(av >= thr[s])) {
                  const int j = t0 + u0 + k;
                  const float4 r = sweep_load_key(tl, u0 + k);
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
                    if (ki[s][K - 1] != 0x7fffffff) {
                      thr[s] = sweep_threshold(kd[s][K - 1], sweep_qq(qx[s], qy[s], qz[s]));
                      if (HALF) thr[s] = fminf(thr[s], pthr[s]);
                    }
                  }
                }
              }
            }
          }
        }
      }
      };
      if constexpr (HALF && FIRSTX) {
        // FIRSTX (key clouds of at most 32 tiles): the lists fill during the first tile, where most
        // insertions happen -- exchange after every 64 keys there, so that no lane goes on with a
        // bound from its own few keys only (16 x 2048 x 8192, k = 3: 0.205 -> 0.173 ms; 4 x 10000 x
        // 512: 0.050 -> 0.040).  A separate instantiation: with long key clouds the first tile does
        // not matter and the second copy of the loop costs the steady state 3 %.
        if (t == 0) {
          for (int c0 = 0; c0 < lim; c0 += 64) {
            sweep(c0, min(lim, c0 + 64));
            exchange();
          }
        } else {
          sweep(0, lim);
        }
      } else {
        sweep(0, lim);
      }
      if (more) {
        float4 *nx = tile[(t + 1) & 1];
#pragma unroll
        for (int p = 0; p < PER; ++p) sweep_store_key(nx, tid + p * KN_THREADS, nxt[p].x, nxt[p].y, nxt[p].z, nxt[p].w);
      }
      if constexpr (HALF) exchange();
      __syncthreads();
    }

    if constexpr (HALF) {
      // merge the lanes' sorted lists by (distance, index) in butterfly steps; every lane ends up
      // with the result
#pragma unroll
      for (int o = QL; o < 32; o <<= 1) {
#pragma unroll
      for (int s = 0; s < Q; ++s) {
        float od_[K];
        int oi_[K];
#pragma unroll
        for (int c = 0; c < K; ++c) {
          od_[c] = __shfl_xor_sync(0xffffffffu, kd[s][c], o);
          oi_[c] = __shfl_xor_sync(0xffffffffu, ki[s][c], o);
        }
        float rd[K];
        int ri[K];
        int pa = 0, pb = 0;
#pragma unroll
        for (int c = 0; c < K; ++c) {
          // heads of the two lists (K is at most 4: the selects below unroll into a few moves)
          float da = pinf(), db = pinf();
          int ia = 0x7fffffff, ib = 0x7fffffff;
#pragma unroll
          for (int e = 0; e < K; ++e) {
            if (e == pa) {
              da = kd[s][e];
              ia = ki[s][e];
            }
            if (e == pb) {
              db = od_[e];
              ib = oi_[e];
            }
          }
          const bool take_a = da < db || (da == db && ia <= ib);
          rd[c] = take_a ? da : db;
          ri[c] = take_a ? ia : ib;
          pa += take_a ? 1 : 0;
          pb += take_a ? 0 : 1;
        }
#pragma unroll
        for (int c = 0; c < K; ++c) {
          kd[s][c] = rd[c];
          ki[s][c] = ri[c];
        }
      }
      }
    }

#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = qindex(s);
      if (i < N1 && half == 0) {
        float *od = dist + (b * N1 + i) * K;
#pragma unroll
        for (int c = 0; c < K; ++c) {
          od[c] = kd[s][c];
          index.put((b * N1 + i) * K + c, ki[s][c]);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
template <int Q>
__global__ void __launch_bounds__(KN_THREADS)
knn_buffered_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2,
                    int k, float *__restrict__ dist, IndexOut index, int64_t blocks_total, XyzLayout ql,
                    XyzLayout kl) {
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
        load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx[s], qy[s], qz[s]);
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
    for (int p = 0; p < PER; ++p) tile[tid + p * KN_THREADS] = make_key(rb, tid + p * KN_THREADS, N2, kl);
    __syncthreads();

    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * KN_TILE;
      const float4 *tl = tile + (t & 1) * KN_TILE;
      const bool more = t + 1 < ntiles;
      float4 nxt[PER];
      if (more) {
#pragma unroll
        for (int p = 0; p < PER; ++p) nxt[p] = make_key(rb, t0 + KN_TILE + tid + p * KN_THREADS, N2, kl);
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
            // d orders before e: smaller, or a number against a NaN (NaN distances order last)
            auto before = [](float x, float e) { return x < e || (e != e && x == x); };
            if (nk[s] == k && !before(d, d_s[(k - 1) * KN_THREADS])) continue;
            int pos = nk[s] < k ? nk[s] : k - 1;
            while (pos > 0 && before(d, d_s[(pos - 1) * KN_THREADS])) {
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
        const float *d_s = ld + ((size_t)s * k) * KN_THREADS + tid;
        const int *i_s = li + ((size_t)s * k) * KN_THREADS + tid;
        for (int c = 0; c < k; ++c) {
          od[c] = d_s[c * KN_THREADS];
          index.put((b * N1 + i) * k + c, i_s[c * KN_THREADS]);
        }
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// Two-pass kernel for 4 < k <= 64 (fp32; larger k: knn_select.cu).
//
// Pass 1 sweeps all keys with the cheap filter value a (3 FMA per pair) and keeps, per query, the
// minimum of a over NCH >= 2k interleaved key classes.  The k-th smallest class minimum tau bounds
// the k-th smallest exact distance from above: the k classes at or below it each hold a distinct key
// with a <= tau, and for any key
//     d <= (a + 22.2u |r|^2 + 3.1u |q|^2 + |q|^2) (1 + 5.1u)
// (upper counterpart of the bound derived in sweep.cuh; |r|^2 <= the cloud's maximum).
// Pass 2 sweeps the keys again and records every GROUP of eight keys whose smallest filter value
// admits d <= that bound -- about 1.3 k groups, nearly all holding a single candidate.  The keys of
// the recorded groups then get their exact distance, the ones below the bound (about 1.35 k) are
// ranked by (distance, index) among themselves and the first k go straight to the output row.
// Nothing data dependent happens inside the sweeps: the group append is six predicated
// straight-line instructions per eight pairs, so the lanes of a warp stay in step whatever the
// insert pattern of a one-pass top-k would look like.
//
// Work split: a block of 4 warps serves 32*Q queries (lane = query) and every warp sweeps a quarter
// of every key tile, so a cloud of a few thousand queries still fills the GPU.  In pass 1 a warp
// takes the key PAIRS w, w + 4, w + 8, ... of a tile (w = its number rotated by the tile number),
// in blocks of NCH/4 pairs that are rotated by the tile number as well, and pair c of the p-th
// block belongs to class (c + p) mod (NCH/4).  Consecutive keys, keys one row apart in a row-major
// depth image and keys of neighbouring tiles thus land in different warps and classes, which
// keeps the bound tight for spatially ordered clouds, whose nearest keys sit close to one another
// in memory (with a plain "position in tile" mapping they share a few classes and the bound
// degenerates).  In pass 2 a warp takes a contiguous quarter of the tile in groups of eight keys.
// Class minima are merged through shared memory: for 32 classes every warp sorts its eight minima
// with a 19-comparator network and one thread per query merges the four sorted runs up to the k-th
// element; for more classes every value is ranked by counting.
// Groups of a query go to ONE list per query (slot claimed with a shared-memory atomic, so the four
// warps share the space and its order is arbitrary).  A group's first candidate replaces the group
// id in its list slot, further candidates of the same group (rare) go behind the list; the exact
// candidate distances reuse the key tiles and class minima (dead by then) -- 31 KB of shared memory
// per block for Q = 2, which keeps seven blocks (28 warps) per SM.
// If a list overflows (massive ties, adversarial or non-finite input) the query falls back to an
// exact scan over all keys by one warp (lanes = keys, sorted list in the query's list column).
constexpr int KT_THREADS = 128;
constexpr int KT_SPLIT = KT_THREADS / 32;  // warps sharing every tile
// KT_NCH key classes (32 to 128: at least two per wanted neighbour, i.e. k <= KT_NCH / 2; a warp
// holds the minima of its KT_NCH / 4 classes in registers) and KT_QCAP group slots per query are
// template parameters of the kernel:
//     k <= 16: 32 classes, 56 slots, one or two queries per lane
//     k <= 32: 64 classes, 104 slots, one query per lane
//     k <= 64: 128 classes, 192 slots, one query per lane
// (KT_TILE = keys per tile: 256.)
template <int Q, int KT_NCH, int KT_QCAP, int KT_TILE>
constexpr size_t kt_smem_bytes() {
  return (size_t)2 * KT_TILE * 16 + (size_t)KT_NCH * 32 * Q * 4 + (size_t)KT_QCAP * 32 * Q * 4;
}

// Predicated append: if a < thr, claim a slot of the query's list and store v there (when the
// slot exists).  Written in PTX so that it stays five straight-line instructions.
template <int STRIDE_BYTES, int KT_QCAP>
__device__ __forceinline__ void kt_append(float a, float thr, unsigned cnt_addr, unsigned cand_addr, int v) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .pred q;\n\t"
      ".reg .s32 sl;\n\t"
      ".reg .u32 ad;\n\t"
      "setp.ltu.f32 p, %0, %1;\n\t"
      "@p atom.shared.add.s32 sl, [%2], 1;\n\t"
      "setp.lt.and.s32 q, sl, %5, p;\n\t"
      "mad.lo.u32 ad, sl, %6, %3;\n\t"
      "@q st.shared.s32 [ad], %4;\n\t"
      "}" ::"f"(a),
      "f"(thr), "r"(cnt_addr), "r"(cand_addr), "r"(v), "n"(KT_QCAP), "n"(STRIDE_BYTES));
}

// Compare-exchange of a sorting network.
__device__ __forceinline__ void kt_cx(float &a, float &b) {
  const float lo = fminf(a, b), hi = fmaxf(a, b);
  a = lo;
  b = hi;
}

// Q = queries per lane (1 or 2): a block serves 32*Q queries.  Two queries per lane halve the
// shared-memory reads per pair, one keeps more blocks in flight when queries are few.
template <int Q, int KT_NCH, int KT_QCAP, int MINB, int KT_TILE>
__global__ void __launch_bounds__(KT_THREADS, MINB)
knn_twopass_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2, int k,
                   float *__restrict__ dist, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  constexpr int PER = KT_TILE / KT_THREADS;
  constexpr int CPW = KT_NCH / KT_SPLIT;          // classes per warp: 8, 16, 32 or 64
  constexpr int NPAIR = KT_TILE / 2 / KT_SPLIT;   // key pairs per warp and tile: 32 or 64
  constexpr int PPC = NPAIR / CPW;                // key pairs per class, tile and warp: 4, 2 or 1
  constexpr int GPP = NPAIR / 4;                  // groups of four pairs (eight keys) per warp and tile
  constexpr int QS = 32 * Q;                      // query slots per block
  constexpr int NSUB = KT_THREADS / QS;           // threads per query in the selection
  constexpr int REGION = 2 * KT_TILE * 16 + KT_NCH * QS * 4;  // bytes of tile + class minima
  constexpr int FCAP = REGION / (QS * 4);         // exact candidate distances that fit into that region
  extern __shared__ __align__(16) unsigned char kt_smem[];
  float4 *tile = reinterpret_cast<float4 *>(kt_smem);                                  // [2][KT_TILE], pair layout
  float *cm = reinterpret_cast<float *>(kt_smem + 2 * KT_TILE * 16);                   // [KT_NCH][QS] class minima
  int *cand = reinterpret_cast<int *>(kt_smem + REGION);                               // [KT_QCAP][QS] group ids
  float *cd = reinterpret_cast<float *>(kt_smem);  // [FCAP][QS] exact distances; reuses tile + cm after pass 2
  static_assert(KT_QCAP >= KT_NCH / 2, "the fallback keeps its k <= KT_NCH / 2 list in the query's own column");
  static_assert(FCAP >= KT_NCH / 2, "and its distances in the query's column of cd");
  static_assert(PPC >= 1 && NPAIR % 4 == 0, "whole classes and whole groups per warp and tile");
  static_assert(FCAP >= KT_QCAP, "a distance slot for every list slot");
  __shared__ int ccnt[QS];  // groups recorded per query (pass 2); later: "needs the exact scan"
  __shared__ int fcnt[QS];  // candidates stored behind the group list
  __shared__ int hcnt[QS];  // candidates found in all
  __shared__ float s_rmax[KT_SPLIT];
  __shared__ float s_tau[QS];  // k-th smallest class minimum; after the thresholds are formed, the bound itself
  const int tid = threadIdx.x, lane = tid & 31, part = tid >> 5;
  const int chunks = (N1 + QS - 1) / QS;
  const float u = 5.9604645e-8f;
  const unsigned cnt_base = (unsigned)__cvta_generic_to_shared(ccnt);
  const unsigned cand_base = (unsigned)__cvta_generic_to_shared(cand);

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int ibase = (int)(blk % chunks) * QS;
    float qx[Q], qy[Q], qz[Q], qq[Q];
    float2 mx[Q], my[Q], mz[Q];
    bool valid[Q];
    __syncthreads();  // the previous iteration's candidate distances alias the tile
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = ibase + s * 32 + lane;
      valid[s] = i < N1;
      qx[s] = qy[s] = qz[s] = 0.f;
      if (valid[s]) load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx[s], qy[s], qz[s]);
      mx[s] = make_float2(-2.f * qx[s], -2.f * qx[s]);
      my[s] = make_float2(-2.f * qy[s], -2.f * qy[s]);
      mz[s] = make_float2(-2.f * qz[s], -2.f * qz[s]);
      qq[s] = sweep_qq(qx[s], qy[s], qz[s]);
    }
    const float *rb = key + b * (int64_t)N2 * 3;
    const int ntiles = (N2 + KT_TILE - 1) / KT_TILE;

    // Key tiles are fetched into registers one tile ahead and committed to the other shared
    // buffer after the current tile has been processed, so global latency overlaps the sweep.
    float rmax = 0.f;
    float4 nxt[PER];
    auto fetch = [&](int t0) {
#pragma unroll
      for (int p = 0; p < PER; ++p) {
        nxt[p] = make_key(rb, t0 + tid + p * KT_THREADS, N2, kl);
        if (t0 + tid + p * KT_THREADS < N2) rmax = fmaxf(rmax, fabsf(nxt[p].w));
      }
    };
    auto commit = [&](float4 *dst) {
#pragma unroll
      for (int p = 0; p < PER; ++p) sweep_store_key(dst, tid + p * KT_THREADS, nxt[p].x, nxt[p].y, nxt[p].z, nxt[p].w);
    };

    // ---- pass 1: minima of the filter value over this warp's classes
    float cmin[Q][CPW];
#pragma unroll
    for (int s = 0; s < Q; ++s)
#pragma unroll
      for (int c = 0; c < CPW; ++c) cmin[s][c] = pinf();
    fetch(0);
    commit(tile);
    __syncthreads();
    for (int t = 0; t < ntiles; ++t) {
      // pair i of this warp sits in float4 slots 2 * (i * KT_SPLIT + w), w = warp rotated by the tile
      const float4 *tl = tile + (t & 1) * KT_TILE + 2 * ((part + t) & (KT_SPLIT - 1));
      if (t + 1 < ntiles) fetch((t + 1) * KT_TILE);
#pragma unroll
      for (int p = 0; p < PPC; ++p) {
        const float4 *tb = tl + 2 * KT_SPLIT * CPW * ((p + t) % PPC);  // block of CPW pairs, rotated too
#pragma unroll
        for (int c = 0; c < CPW; ++c) {
          const float4 A = tb[2 * KT_SPLIT * c], Bv = tb[2 * KT_SPLIT * c + 1];
          const float2 kx = make_float2(A.x, A.y), ky = make_float2(A.z, A.w);
          const float2 kz = make_float2(Bv.x, Bv.y), kw = make_float2(Bv.z, Bv.w);
#pragma unroll
          for (int s = 0; s < Q; ++s) {
            const float2 a = __ffma2_rn(mx[s], kx, __ffma2_rn(my[s], ky, __ffma2_rn(mz[s], kz, kw)));
            cmin[s][(c + p) % CPW] = sweep_min3(cmin[s][(c + p) % CPW], a.x, a.y);
          }
        }
      }
      if (t + 1 < ntiles) commit(tile + ((t + 1) & 1) * KT_TILE);
      __syncthreads();
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    if (lane == 0) s_rmax[part] = rmax;
    if (tid < QS) s_tau[tid] = pinf();

    // ---- k-th smallest class minimum of each query
    if constexpr (CPW == 8) {
      // every warp sorts its eight minima (19 compare-exchanges) ...
#pragma unroll
      for (int s = 0; s < Q; ++s) {
        float(&v)[CPW] = cmin[s];
        kt_cx(v[0], v[1]); kt_cx(v[2], v[3]); kt_cx(v[4], v[5]); kt_cx(v[6], v[7]);
        kt_cx(v[0], v[2]); kt_cx(v[1], v[3]); kt_cx(v[4], v[6]); kt_cx(v[5], v[7]);
        kt_cx(v[1], v[2]); kt_cx(v[5], v[6]); kt_cx(v[0], v[4]); kt_cx(v[3], v[7]);
        kt_cx(v[1], v[5]); kt_cx(v[2], v[6]);
        kt_cx(v[1], v[4]); kt_cx(v[3], v[6]);
        kt_cx(v[2], v[4]); kt_cx(v[3], v[5]);
        kt_cx(v[3], v[4]);
#pragma unroll
        for (int c = 0; c < CPW; ++c) cm[(part * CPW + c) * QS + s * 32 + lane] = v[c];
      }
      __syncthreads();
      // ... and one thread per query merges the four sorted runs up to the k-th element
      if (tid < QS) {
        static_assert(KT_SPLIT == 4, "four sorted runs");
        const float *run = cm + tid;  // element e of run w: run[(w * CPW + e) * QS]
        int p0 = 0, p1 = 0, p2 = 0, p3 = 0;
        float h0 = run[0], h1 = run[CPW * QS], h2 = run[2 * CPW * QS], h3 = run[3 * CPW * QS];
        float v = pinf();
        for (int r = 0; r < k; ++r) {
          // the smallest head leaves its run (the first such run on equal values); written without
          // branches: every head is re-read from its run's current position
          v = fminf(fminf(h0, h1), fminf(h2, h3));
          const bool t0 = h0 == v, t1 = !t0 && h1 == v, t2 = !t0 && !t1 && h2 == v, t3 = !t0 && !t1 && !t2 && h3 == v;
          p0 += t0 ? 1 : 0;
          p1 += t1 ? 1 : 0;
          p2 += t2 ? 1 : 0;
          p3 += t3 ? 1 : 0;
          const float n0 = run[min(p0, CPW - 1) * QS], n1 = run[(CPW + min(p1, CPW - 1)) * QS];
          const float n2 = run[(2 * CPW + min(p2, CPW - 1)) * QS], n3 = run[(3 * CPW + min(p3, CPW - 1)) * QS];
          h0 = p0 < CPW ? n0 : pinf();
          h1 = p1 < CPW ? n1 : pinf();
          h2 = p2 < CPW ? n2 : pinf();
          h3 = p3 < CPW ? n3 : pinf();
        }
        s_tau[tid] = v;
      }
      __syncthreads();
    } else {
#pragma unroll
      for (int s = 0; s < Q; ++s)
#pragma unroll
        for (int c = 0; c < CPW; ++c) cm[(part * CPW + c) * QS + s * 32 + lane] = cmin[s][c];
      __syncthreads();
      // rank by counting (ties broken by class number); the value with rank k-1 is published
#pragma unroll
      for (int s = 0; s < Q; ++s) {
#pragma unroll
        for (int c = 0; c < CPW; ++c) {
          const float v = cmin[s][c];
          const int cc = part * CPW + c;
          int rank = 0;
#pragma unroll 8
          for (int o = 0; o < KT_NCH; ++o) {
            const float w = cm[o * QS + s * 32 + lane];
            rank += (w < v || (w == v && o < cc)) ? 1 : 0;
          }
          if (rank == k - 1) s_tau[s * 32 + lane] = v;
        }
      }
      __syncthreads();
    }
    rmax = fmaxf(fmaxf(s_rmax[0], s_rmax[1]), fmaxf(s_rmax[2], s_rmax[3]));
    // Upper bound of the k-th smallest exact distance (constants rounded up generously to cover
    // the roundings of this very computation), then the filter threshold that admits every key
    // at or below it.  Anything non-finite sends the query to the exact fallback: its counter
    // starts beyond the capacity and its threshold admits nothing.
    float thr[Q], lim[Q];
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const float tau = s_tau[s * 32 + lane];
      const float a_up = tau + 32.f * u * rmax + 8.f * u * qq[s];
      const float d_up = (a_up + qq[s] * (1.f + 8.f * u)) * (1.f + 10.f * u) + 1e-37f;
      lim[s] = __int_as_float(__float_as_int(fmaxf(d_up, 0.f)) + 1);  // next float up
      const bool finite = d_up < 3.0e38f && rmax < 1.0e30f && qq[s] < 1.0e30f;
      thr[s] = (finite && valid[s]) ? sweep_threshold(lim[s], qq[s]) : -pinf();
      if (part == 0) {
        ccnt[s * 32 + lane] = (finite || !valid[s]) ? 0 : KT_QCAP + 1;
        fcnt[s * 32 + lane] = 0;
        hcnt[s * 32 + lane] = 0;
      }
    }

    // ---- pass 2: record the groups of eight consecutive keys (group id = first key / 8) that hold
    // a candidate; padding keys carry w = +inf and never pass.
    fetch(0);
    commit(tile);
    __syncthreads();
    if (part == 0) {  // every warp has read s_tau by now: it carries the bound from here on
#pragma unroll
      for (int s = 0; s < Q; ++s) s_tau[s * 32 + lane] = lim[s];
    }
    for (int t = 0; t < ntiles; ++t) {
      const float4 *tl = tile + (t & 1) * KT_TILE + part * (KT_TILE / KT_SPLIT);
      const int g0 = (t * KT_TILE + part * (KT_TILE / KT_SPLIT)) >> 3;
      if (t + 1 < ntiles) fetch((t + 1) * KT_TILE);
#pragma unroll 2
      for (int g = 0; g < GPP; ++g) {
        float2 a[4][Q];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float4 A = tl[8 * g + 2 * p], Bv = tl[8 * g + 2 * p + 1];
          const float2 kx = make_float2(A.x, A.y), ky = make_float2(A.z, A.w);
          const float2 kz = make_float2(Bv.x, Bv.y), kw = make_float2(Bv.z, Bv.w);
#pragma unroll
          for (int s = 0; s < Q; ++s)
            a[p][s] = __ffma2_rn(mx[s], kx, __ffma2_rn(my[s], ky, __ffma2_rn(mz[s], kz, kw)));
        }
#pragma unroll
        for (int s = 0; s < Q; ++s) {
          float m = sweep_min3(a[0][s].x, a[0][s].y, a[1][s].x);
          m = sweep_min3(m, a[1][s].y, a[2][s].x);
          m = sweep_min3(m, a[2][s].y, a[3][s].x);
          m = fminf(m, a[3][s].y);
          kt_append<QS * 4, KT_QCAP>(m, thr[s], cnt_base + 4u * (s * 32 + lane), cand_base + 4u * (s * 32 + lane),
                                     g0 + g);
        }
      }
      if (t + 1 < ntiles) commit(tile + ((t + 1) & 1) * KT_TILE);
      __syncthreads();
    }

    // ---- exact selection: NSUB threads per query.  The eight keys of every recorded group get
    // their exact distance (all 24 coordinates are loaded before any is used, so the loads of a
    // group overlap); keys below the bound are the candidates.  A group's first candidate takes
    // the group's own list slot (distance in cd, key index in cand; -1 / +inf when the group holds
    // none), any further ones go behind the list.  Then each candidate is ranked by (distance,
    // index) among its query's candidates and ranks below k go straight to the output row.
    const int col = tid % QS, sub = tid / QS;
    const int iq = ibase + col;
    const bool qvalid = iq < N1;
    const int n = ccnt[col];
    float cqx = 0.f, cqy = 0.f, cqz = 0.f;
    if (qvalid) load_xyz(query + b * 3 * (int64_t)N1, iq, ql, cqx, cqy, cqz);
    if (qvalid && n <= KT_QCAP) {
      const float bound = s_tau[col];
      int hits = 0;
      // [N,3] clouds whose rows start on 16-byte boundaries: a whole group is six 16-byte loads
      const bool vec = kl.cs == 1 && (reinterpret_cast<uintptr_t>(rb) & 15) == 0;
      for (int c = sub; c < n; c += NSUB) {
        const int j0 = cand[c * QS + col] * 8;
        float rx[8], ry[8], rz[8];
        if (vec && j0 + 8 <= N2) {
          const float4 *g4 = reinterpret_cast<const float4 *>(rb + (int64_t)j0 * 3);
          const float4 v0 = __ldg(g4), v1 = __ldg(g4 + 1), v2 = __ldg(g4 + 2), v3 = __ldg(g4 + 3), v4 = __ldg(g4 + 4),
                       v5 = __ldg(g4 + 5);
          rx[0] = v0.x, ry[0] = v0.y, rz[0] = v0.z, rx[1] = v0.w, ry[1] = v1.x, rz[1] = v1.y;
          rx[2] = v1.z, ry[2] = v1.w, rz[2] = v2.x, rx[3] = v2.y, ry[3] = v2.z, rz[3] = v2.w;
          rx[4] = v3.x, ry[4] = v3.y, rz[4] = v3.z, rx[5] = v3.w, ry[5] = v4.x, rz[5] = v4.y;
          rx[6] = v4.z, ry[6] = v4.w, rz[6] = v5.x, rx[7] = v5.y, ry[7] = v5.z, rz[7] = v5.w;
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) load_xyz(rb, min(j0 + e, N2 - 1), kl, rx[e], ry[e], rz[e]);
        }
        int first = -1;
        float firstd = pinf();
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = sqdist<float>(rx[e], ry[e], rz[e], cqx, cqy, cqz);
          if (j0 + e < N2 && d < bound) {
            ++hits;
            if (first < 0) {
              first = j0 + e;
              firstd = d;
            } else {
              const int row = n + atomicAdd(&fcnt[col], 1);
              if (row < KT_QCAP) {
                cd[row * QS + col] = d;
                cand[row * QS + col] = j0 + e;
              }
            }
          }
        }
        cd[c * QS + col] = firstd;
        cand[c * QS + col] = first;
      }
      if (hits) atomicAdd(&hcnt[col], hits);
    }
    __syncthreads();
    // A list that overflowed, or -- which the bound derivation rules out for finite input, but which
    // costs nothing to guard -- holds fewer than k candidates, sends its query to the exact scan.
    const int rows = n + fcnt[col];
    const bool listed = n <= KT_QCAP && rows <= KT_QCAP && hcnt[col] >= k;
    if (qvalid && listed) {
      float *od = dist + (b * N1 + iq) * (int64_t)k;
      const int64_t orow = (b * N1 + iq) * (int64_t)k;
      for (int f = sub; f < rows; f += NSUB) {
        const int j = cand[f * QS + col];
        if (j < 0) continue;
        const float d = cd[f * QS + col];
        // rank = candidates with a smaller distance; equal distances (rare) are settled by index
        int rank = 0, same = 0;
#pragma unroll 8
        for (int o = 0; o < rows; ++o) {
          const float w = cd[o * QS + col];  // empty slots hold +inf
          rank += w < d ? 1 : 0;
          same += w == d ? 1 : 0;
        }
        if (same > 1) {
          for (int o = 0; o < rows; ++o)
            rank += (cd[o * QS + col] == d && (unsigned)cand[o * QS + col] < (unsigned)j) ? 1 : 0;  // -1 is last
        }
        if (rank < k) {
          od[rank] = d;
          index.put(orow + rank, j);
        }
      }
    }
    __syncthreads();  // every thread is done with the lists before an exact scan reuses a column
    if (sub == 0) ccnt[col] = (qvalid && !listed) ? 1 : 0;
    __syncthreads();

    // ---- exact scan of the queries flagged above, one warp per query: lanes take 32 consecutive
    // keys at a time; a key that beats the current k-th entry is inserted into the sorted list kept
    // in the first k slots of the query's own column of cd / cand (position by counting, entries
    // behind it moved up by the lanes together).  Keys arrive in ascending index order, so a key
    // equal to the k-th distance never enters a full list and equal distances stay in index order.
    // A NaN distance counts as +inf for the ordering.
    for (int fc = part; fc < QS; fc += KT_SPLIT) {
      if (ccnt[fc] == 0) continue;  // uniform over the warp
      const int fq = ibase + fc;
      float fx, fy, fz;
      load_xyz(query + b * 3 * (int64_t)N1, fq, ql, fx, fy, fz);
      int nk = 0;
      float kth = pinf();
      for (int base = 0; base < N2; base += 32) {
        const int j = base + lane;
        float d = pinf();
        if (j < N2) {
          float rx, ry, rz;
          load_xyz(rb, j, kl, rx, ry, rz);
          d = sqdist<float>(rx, ry, rz, fx, fy, fz);
        }
        const float dv = d == d ? d : pinf();  // ordering value
        unsigned mask = __ballot_sync(0xffffffffu, j < N2 && (nk < k || dv < kth));
        while (mask) {
          const int l = __ffs(mask) - 1;
          mask &= mask - 1;
          const float dn = __shfl_sync(0xffffffffu, d, l), dnv = __shfl_sync(0xffffffffu, dv, l);
          if (nk == k && !(dnv < kth)) continue;  // the k-th entry tightened since the ballot
          // position: entries ordering at or before the new key (equal distances hold lower indices)
          int before = 0;
          for (int r = lane; r < nk; r += 32) {
            const float w = cd[r * QS + fc];
            before += ((w == w ? w : pinf()) <= dnv) ? 1 : 0;
          }
          const int pos = __reduce_add_sync(0xffffffffu, before);
          const int last = nk < k ? nk : k - 1;  // slot that receives the old entry last - 1
          // move entries [pos, last) up by one: read them all, then write them all
          float mv[4];
          int mj[4];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int r = lane + 32 * q4;
            if (r >= pos && r < last) {
              mv[q4] = cd[r * QS + fc];
              mj[q4] = cand[r * QS + fc];
            }
          }
          __syncwarp();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int r = lane + 32 * q4;
            if (r >= pos && r < last) {
              cd[(r + 1) * QS + fc] = mv[q4];
              cand[(r + 1) * QS + fc] = mj[q4];
            }
          }
          if (lane == 0) {
            cd[pos * QS + fc] = dn;
            cand[pos * QS + fc] = base + l;
          }
          __syncwarp();
          if (nk < k) ++nk;
          if (nk == k) {
            const float w = cd[(k - 1) * QS + fc];
            kth = w == w ? w : pinf();
          }
        }
      }
      float *od = dist + (b * N1 + fq) * (int64_t)k;
      const int64_t orow = (b * N1 + fq) * (int64_t)k;
      for (int c = lane; c < k; c += 32) {
        od[c] = cd[c * QS + fc];
        index.put(orow + c, cand[c * QS + fc]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Generic kernel (any floating type, any k): one query per thread, exact distances, key tiles in
// shared memory.  The k best so far live in the query's output row as a binary MAX-HEAP ordered by
// (distance, index): the root is the current k-th neighbour, a key enters only if it beats the root
// (keys arrive in ascending index order, so "d < root distance" is the whole test), replaces it and
// sifts down in O(log k) steps -- the reference rescans all k entries for every accepted key.  At
// the end the heap is turned into an ascending row by heap sort.
// (v, jv) orders after (m, jm): by distance, then index; a NaN distance orders after every number.
template <typename T>
__device__ __forceinline__ bool knn_larger(T v, int64_t jv, T m, int64_t jm) {
  const bool vn = !(v == v), mn = !(m == m);
  if (vn != mn) return vn;
  if (vn) return jv > jm;
  return v > m || (v == m && jv > jm);
}

// Sift (d, j) down from the root of the max-heap od[0, n) / oi[row, row + n).
template <typename T>
__device__ __forceinline__ void knn_sift_down(T *__restrict__ od, IndexOut oi, int64_t row, int64_t n, T d,
                                              int64_t j) {
  int64_t pos = 0;
  while (true) {
    int64_t child = 2 * pos + 1;
    if (child >= n) break;
    T dc = od[child];
    int64_t jc = oi.get(row + child);
    if (child + 1 < n) {
      const T dr = od[child + 1];
      const int64_t jr = oi.get(row + child + 1);
      if (knn_larger<T>(dr, jr, dc, jc)) {
        ++child;
        dc = dr;
        jc = jr;
      }
    }
    if (!knn_larger<T>(dc, jc, d, j)) break;
    od[pos] = dc;
    oi.put(row + pos, jc);
    pos = child;
  }
  od[pos] = d;
  oi.put(row + pos, j);
}

// Blocks of 64 threads: the per-query work is long and serial, so many small blocks keep every SM
// busy even for a few thousand queries.
constexpr int KG_THREADS = 64;
template <typename T>
__global__ void __launch_bounds__(KG_THREADS)
knn_generic_kernel(const T *__restrict__ query, const T *__restrict__ key, int64_t B, int64_t N1, int64_t N2,
                   int64_t k, T *__restrict__ dist, IndexOut oi, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  constexpr int TILE = KG_THREADS;
  static_assert((TILE & (TILE - 1)) == 0 && TILE % 8 == 0, "tile indices are masked; batches of eight");
  __shared__ T sx[TILE], sy[TILE], sz[TILE];
  const int tid = threadIdx.x;
  if (blockIdx.x < blocks_total) {  // defined contents for the slots a short first tile leaves unwritten
    sx[tid] = 0;
    sy[tid] = 0;
    sz[tid] = 0;
  }
  __syncthreads();
  const int64_t chunks = (N1 + TILE - 1) / TILE;
  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int64_t i = (blk % chunks) * TILE + tid;
    const bool valid = i < N1;
    T qx = 0, qy = 0, qz = 0;
    if (valid) load_xyz(query + b * 3 * N1, i, ql, qx, qy, qz);
    T *od = dist + (b * N1 + (valid ? i : 0)) * k;
    const int64_t row = (b * N1 + (valid ? i : 0)) * k;  // offset of this query's index row
    int64_t cnt = 0;
    T root = Exact<T>::inf();  // distance at the heap's root once the heap is full
    const T *rb = key + b * N2 * 3;
    for (int64_t t0 = 0; t0 < N2; t0 += TILE) {
      const int64_t jl = t0 + tid;
      if (jl < N2) load_xyz(rb, jl, kl, sx[tid], sy[tid], sz[tid]);
      __syncthreads();
      const int lim = (int)((N2 - t0) < TILE ? (N2 - t0) : TILE);
      if (valid) {
        // Eight distances at a time: with one or two warps per SM sub-partition the loop is bound
        // by the latency of the dependent arithmetic, which independent chains hide.  (Slots beyond
        // lim hold stale coordinates; their distances are computed and ignored.)
        for (int u0 = 0; u0 < lim; u0 += 8) {
          T dd[8];
#pragma unroll
          for (int w = 0; w < 8; ++w) dd[w] = sqdist<T>(sx[(u0 + w) & (TILE - 1)], sy[(u0 + w) & (TILE - 1)],
                                                        sz[(u0 + w) & (TILE - 1)], qx, qy, qz);
#pragma unroll
          for (int w = 0; w < 8; ++w) {
            const T d = dd[w];
            const int64_t j = t0 + u0 + w;
            if (u0 + w >= lim) break;
            if (cnt < k) {
              // filling: sift the new element UP from the end of the heap
              int64_t pos = cnt++;
              while (pos > 0) {
                const int64_t par = (pos - 1) >> 1;
                const T dp = od[par];
                const int64_t jp = oi.get(row + par);
                if (!knn_larger<T>(d, j, dp, jp)) break;
                od[pos] = dp;
                oi.put(row + pos, jp);
                pos = par;
              }
              od[pos] = d;
              oi.put(row + pos, j);
              if (cnt == k) root = od[0];
            } else if (d < root || (root != root && d == d)) {
              // a key enters when it beats the root; a NaN at the root (it orders after every
              // number) gives way to any real distance
              knn_sift_down<T>(od, oi, row, k, d, j);
              root = od[0];
            }
          }
        }
      }
      __syncthreads();
    }
    if (valid) {
      // heap sort: move the largest to the end, restore the heap on the shorter prefix
      for (int64_t end = cnt - 1; end > 0; --end) {
        const T dl = od[end];
        const int64_t jl2 = oi.get(row + end);
        od[end] = od[0];
        oi.put(row + end, oi.get(row));
        knn_sift_down<T>(od, oi, row, end, dl, jl2);
      }
    }
  }
}

// Arguments every launcher passes on unchanged: output index tensor (int64 or int32) and the
// coordinate layouts of the query and key clouds.
struct KnnIo {
  IndexOut index;
  XyzLayout ql, kl;
};

template <typename T>
int knn_generic(const T *query, const T *key, int64_t B, int64_t N1, int64_t N2, int64_t k, T *dist, const KnnIo &io,
                cudaStream_t st) {
  const int64_t total = B * ((N1 + KG_THREADS - 1) / KG_THREADS);
  if (total == 0) return TK3D_OK;
  const int64_t cap = (int64_t)sm_count() * 256;
  knn_generic_kernel<T><<<(unsigned)(total < cap ? total : cap), KG_THREADS, 0, st>>>(query, key, B, N1, N2, k, dist,
                                                                                     io.index, total, io.ql, io.kl);
  return check_launch("knn_generic_kernel");
}

template <int K, int Q, int LANES = 1>
int knn_small(const float *query, const float *key, int64_t B, int N1, int N2, float *dist, const KnnIo &io,
              cudaStream_t st) {
  const int64_t per = KN_THREADS * Q / LANES;
  const int64_t total = B * ((N1 + per - 1) / per);
  const int64_t cap = (int64_t)sm_count() * 256;
  const unsigned grid = (unsigned)(total < cap ? total : cap);
  if (LANES > 1 && N2 <= 16384)  // few key tiles: the first one is worth extra exchanges
    knn_small_kernel<K, Q, LANES, (LANES > 1)><<<grid, KN_THREADS, 0, st>>>(query, key, B, N1, N2, dist, io.index, total,
                                                                            io.ql, io.kl);
  else
    knn_small_kernel<K, Q, LANES><<<grid, KN_THREADS, 0, st>>>(query, key, B, N1, N2, dist, io.index, total, io.ql,
                                                               io.kl);
  return check_launch("knn_small_kernel");
}

// Lanes per query for launches with one query per thread (fewer than about 75 000 queries).  Measured
// on B200 (148 SMs), k = 1 / k = 3, in ms:
//   queries   1 lane        2 lanes       4 lanes       8 lanes        (queries x keys)
//   65536     0.35 / 0.48   0.31 / 0.44   0.57 / 0.64   1.13 / 1.18    4 x 16384 x 16384
//   65536     0.109/ 0.192  0.096/ 0.200  0.166/ 0.220  0.304/ 0.352   1 x 65536 x 4096
//   40000     0.029/ 0.057  0.029/ 0.049  0.028/ 0.056  0.040/ 0.063   4 x 10000 x 512
//   32768     0.039/ 0.079  0.033/ 0.067  0.031/ 0.053  0.054/ 0.074   32 x 1024 x 1024
//   32768                   0.118/ 0.202  0.151/ 0.185  0.291/ 0.319   16 x 2048 x 8192
//   16384     0.055/ 0.112  0.041/ 0.077  0.034/ 0.055  0.046/ 0.057   8 x 2048 x 2048
//    8192     0.43 / 0.64   0.28 / 0.32   0.21 / 0.24   0.33 / 0.35    2 x 4096 x 32768
//    4096                   0.52 / 0.54   0.34 / 0.37   0.38 / 0.39    1 x 4096 x 65536
//    2048     0.159/ 0.276  0.108/ 0.156  0.071/ 0.100  0.054/ 0.072   4 x 512 x 10000
//    1000     1.16 / 1.58   0.76 / 0.74   0.51 / 0.52   0.40 / 0.43    1 x 1000 x 100000
inline int lanes_per_query(int64_t nq) {
  const int64_t sms = sm_count();
  if (nq * 6 > sms * 1000) return 2;   // above about 24 600 queries on 148 SMs
  if (nq * 48 > sms * 1000) return 4;  // above about 3 000
  return 8;
}

template <int K>
int knn_small_q(const float *query, const float *key, int64_t B, int N1, int N2, float *dist, const KnnIo &io,
                cudaStream_t st) {
  const int64_t sms = sm_count();
  const int64_t nq = B * (int64_t)N1;
  // At most half a round of 256-query tasks (seven per SM make a round): two lanes per query, i.e.
  // twice the warps and still one round (C5's query slab of an 8-GPU run, 8 x 16384 x 32768: 1.16 ->
  // 1.07 ms; 16 x 8192 x 8192, k = 1: 0.29 -> 0.25 ms).  Closer to a full round the doubled tasks spill
  // into a second one (8 x 32000 x 32768, k = 3: 1.81 -> 2.03 ms), so those stay as they are.  With k = 4
  // the two-lane variant needs 79 registers, six blocks per SM instead of seven, and loses (the same
  // slab: 1.64 ms with one lane, 2.34 with two; 1.83 with two capped at 72 registers).
  if (K <= 3 && nq >= sms * 2 * KN_THREADS * 2 && 2 * nq <= sms * 7 * KN_THREADS * 2)
    return knn_small<K, 2, 2>(query, key, B, N1, N2, dist, io, st);
  if (nq >= sms * 2 * KN_THREADS * 2) return knn_small<K, 2>(query, key, B, N1, N2, dist, io, st);
  switch (lanes_per_query(nq)) {
    case 8: return knn_small<K, 1, 8>(query, key, B, N1, N2, dist, io, st);
    case 4: return knn_small<K, 1, 4>(query, key, B, N1, N2, dist, io, st);
    case 2: return knn_small<K, 1, 2>(query, key, B, N1, N2, dist, io, st);
    default: return knn_small<K, 1>(query, key, B, N1, N2, dist, io, st);
  }
}

size_t buffered_smem(int Q, int k) {
  return (size_t)2 * KN_TILE * 16 + (size_t)Q * k * KN_THREADS * 8 + (size_t)Q * KN_CAP * KN_THREADS * 4;
}

template <int Q>
int knn_buffered(const float *query, const float *key, int64_t B, int N1, int N2, int k, float *dist,
                 const KnnIo &io, cudaStream_t st) {
  const int64_t per = KN_THREADS * Q;
  const int64_t total = B * ((N1 + per - 1) / per);
  const size_t smem = buffered_smem(Q, k);
  TK3D_CUDA(raise_smem_limit((const void *)knn_buffered_kernel<Q>, (int)smem));
  const int64_t cap = (int64_t)sm_count() * 64;
  knn_buffered_kernel<Q><<<(unsigned)(total < cap ? total : cap), KN_THREADS, smem, st>>>(
      query, key, B, N1, N2, k, dist, io.index, total, io.ql, io.kl);
  return check_launch("knn_buffered_kernel");
}

template <int Q, int NCH, int QCAP, int MINB, int TILE = 256>
int knn_twopass(const float *query, const float *key, int64_t B, int N1, int N2, int k, float *dist, const KnnIo &io,
                cudaStream_t st) {
  const int64_t total = B * ((N1 + 32 * Q - 1) / (32 * Q));
  const int64_t gcap = (int64_t)sm_count() * 256;
  const size_t smem = kt_smem_bytes<Q, NCH, QCAP, TILE>();
  if (smem + 4096 > 48 * 1024)  // static shared memory of the kernel counts towards the 48 KB default limit
    TK3D_CUDA(raise_smem_limit((const void *)knn_twopass_kernel<Q, NCH, QCAP, MINB, TILE>, (int)smem));
  knn_twopass_kernel<Q, NCH, QCAP, MINB, TILE><<<(unsigned)(total < gcap ? total : gcap), KT_THREADS, smem, st>>>(
      query, key, B, N1, N2, k, dist, io.index, total, io.ql, io.kl);
  return check_launch("knn_twopass_kernel");
}

}  // namespace

// Three nearest keys of every query with inverse-distance weights, the front end of feature
// interpolation: w_i = (1/max(d_i, eps)) / sum_j (1/max(d_j, eps)) and 32-bit indices; N2 >= 3.
// The sweep writes the squared distances into `weight` and a second, tiny kernel turns every row
// into weights in place (0.01 ms for 524288 queries).  Computing the weights in the sweep's own
// epilogue saved that launch but left the sweep's two-lane variant with 79 registers, six blocks
// per SM, i.e. out of reach for the half-filled launches that need it (8 x 16384 x 32768 with the
// gather that follows: 1.24 -> 1.11 ms; 8 x 65536 x 32768: 6.80 -> 6.77).
__global__ void __launch_bounds__(256)
three_nn_weight_inplace_kernel(float *__restrict__ weight, int64_t rows, float eps) {
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
    float *w = weight + r * 3;
    float inv[3], sum = 0.f;
#pragma unroll
    for (int c = 0; c < 3; ++c) {
      inv[c] = __fdiv_rn(1.0f, fmaxf(w[c], eps));
      sum = c == 0 ? inv[0] : __fadd_rn(sum, inv[c]);
    }
#pragma unroll
    for (int c = 0; c < 3; ++c) w[c] = __fdiv_rn(inv[c], sum);
  }
}

int three_nn_fused_f32(const float *query, const float *key, int64_t B, int64_t N1, int64_t N2, int channel_first,
                       float eps, float *weight, int32_t *index32, cudaStream_t st) {
  if (B * N1 == 0) return TK3D_OK;
  KnnIo io;
  io.index = index_out(index32, 1, B * N1 * 3);
  io.ql = xyz_layout(channel_first, N1);
  io.kl = xyz_layout(channel_first, N2);
  int rc = knn_small_q<3>(query, key, B, (int)N1, (int)N2, weight, io, st);
  if (rc) return rc;
  const int64_t rows = B * N1, blocks = (rows + 255) / 256, cap = (int64_t)sm_count() * 8;
  three_nn_weight_inplace_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, st>>>(weight, rows, eps);
  return check_launch("three_nn_weight_inplace_kernel");
}

}  // namespace tk3d

namespace tk3d {
// Radix selection (knn_select.cu): float32, k <= 256.
int knn_select_f32(const float *query, const float *key, int64_t B, int N1, int N2, int k, float *dist, IndexOut index,
                   XyzLayout ql, XyzLayout kl, cudaStream_t st);

bool knn_split_f64(const double *query, const double *key, int64_t B, int64_t N1, int64_t N2, int64_t k, double *dist,
                   IndexOut index, XyzLayout ql, XyzLayout kl, cudaStream_t st, int *rc);
}

using namespace tk3d;

static int knn_impl(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, int64_t k,
                    int channel_first, void *distance, void *index, int index32, int dtype, void *stream) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "knn: dtype %d", dtype);
  TK3D_REQUIRE(B >= 0 && N1 >= 0 && N2 >= 0, TK3D_ERR_SHAPE, "knn: negative size");
  TK3D_REQUIRE(k >= 1, TK3D_ERR_K, "knn: k must be >= 1 (got %lld)", (long long)k);
  TK3D_REQUIRE(N2 >= k, TK3D_ERR_K, "knn: k=%lld exceeds the %lld key points", (long long)k, (long long)N2);
  TK3D_REQUIRE(N1 < (1LL << 30) && N2 < (1LL << 30), TK3D_ERR_SHAPE, "knn: clouds limited to 2^30 points");
  if (B * N1 == 0) return TK3D_OK;
  TK3D_REQUIRE(query && key && distance && index, TK3D_ERR_NULL, "knn: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  KnnIo io;
  io.index = index_out(index, index32, B * N1 * k);
  io.ql = xyz_layout(channel_first, N1);
  io.kl = xyz_layout(channel_first, N2);
  if (dtype == TK3D_F64) {
    int rc = TK3D_OK;  // few queries and k <= 64: several warps per query group (knn_split.cu)
    if (knn_split_f64((const double *)query, (const double *)key, B, N1, N2, k, (double *)distance, io.index, io.ql,
                      io.kl, st, &rc))
      return rc;
    return knn_generic<double>((const double *)query, (const double *)key, B, N1, N2, k, (double *)distance, io, st);
  }
  const float *q = (const float *)query, *r = (const float *)key;
  float *d = (float *)distance;
  switch (k) {
    case 1: return knn_small_q<1>(q, r, B, (int)N1, (int)N2, d, io, st);
    case 2: return knn_small_q<2>(q, r, B, (int)N1, (int)N2, d, io, st);
    case 3: return knn_small_q<3>(q, r, B, (int)N1, (int)N2, d, io, st);
    case 4: return knn_small_q<4>(q, r, B, (int)N1, (int)N2, d, io, st);
    default: break;
  }
  // Two-pass selection needs at least two key classes per wanted neighbour to be tight (the class
  // counts below) and a few keys in every class: N2 >= 4 k, at least 256.
  // Measured on B200 (16 x 4096 x 4096): the two-pass kernel 0.74 ms at k = 64, 2.04 at 100, 2.52 at
  // 128; radix selection (knn_select.cu) 0.82 ms at k = 81, 0.85 at 100, 1.4 at 128 to 240.
  // With fewer than 16 keys per wanted neighbour the class minima stop bounding anything for
  // k > 40 (16 x 4096 x 300, k = 64: 0.47 ms two-pass, 0.26 ms by radix).
  const bool by_radix = (k > 64 || (k > 40 && N2 < 16 * k)) && k <= 256 && N2 < (1LL << 31);
  if (!by_radix && k <= 64 && N2 >= 4 * k && N2 >= 256) {
    if (k <= 16) {
      if (B * N1 >= (int64_t)sm_count() * 4 * 64)
        return knn_twopass<2, 32, 56, 7>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
      return knn_twopass<1, 32, 56, 7>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
    }
    if (k <= 32) return knn_twopass<1, 64, 104, 5>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
    return knn_twopass<1, 128, 192, 4>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
  }
  // key clouds too small for the two-pass kernel: buffered lists up to k = 40 (16 x 4096 x 300:
  // 0.069 ms at k = 16 against 0.195 by radix, 0.47 against 0.26 at k = 64)
  if (k <= 40) {
    const int64_t sms = sm_count();
    if (k <= 32 && B * N1 >= sms * 2 * KN_THREADS * 2)
      return knn_buffered<2>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
    return knn_buffered<1>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
  }
  if (k <= 256 && N2 < (1LL << 31))  // large k: selection by radix, no insertions
    return knn_select_f32(q, r, B, (int)N1, (int)N2, (int)k, d, io.index, io.ql, io.kl, st);
  return knn_generic<float>(q, r, B, N1, N2, k, d, io, st);
}

extern "C" int tk3d_knn(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, int64_t k,
                        void *distance, int64_t *index, int dtype, void *stream) {
  TK3D_RANGE("tk3d_knn");
  return knn_impl(query, key, B, N1, N2, k, 0, distance, index, 0, dtype, stream);
}

extern "C" int tk3d_knn_layout(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, int64_t k,
                               int xyz_channel_first, void *distance, void *index, int index_dtype, int dtype,
                               void *stream) {
  TK3D_RANGE("tk3d_knn_layout");
  TK3D_REQUIRE(index_dtype == TK3D_I64 || index_dtype == TK3D_I32, TK3D_ERR_DTYPE, "knn: index_dtype %d", index_dtype);
  return knn_impl(query, key, B, N1, N2, k, xyz_channel_first != 0, distance, index, index_dtype == TK3D_I32, dtype,
                  stream);
}

TK3D_BOUNDS_TU(knn)
