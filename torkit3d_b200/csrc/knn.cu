// Brute-force k nearest neighbours (squared distances, rows sorted ascending by (distance, index)).
//
// Four kernels:
//   knn_small_kernel<K,Q>  fp32, k <= 4: per-thread top-K in registers, filter-then-verify sweep
//                          (sweep.cuh), insertion straight from the verify branch.  With k << N2
//                          the branch is rare (about k ln(N2/k) times per query).
//   knn_twopass_kernel     fp32, 4 < k <= 128 (and N2 >= 4 k, at least 256): pass 1 bounds the k-th distance from
//                          class minima of the filter value, pass 2 collects the few candidates
//                          below the bound, exact selection among them (see the kernel's header).
//   knn_buffered_kernel<Q> fp32, other k <= 128 (small key clouds): same filter, but passing keys are only appended
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

// ---------------------------------------------------------------------------------------------
// FUSED (three-nearest-neighbour front end of feature interpolation): instead of distances and
// 64-bit indices the epilogue writes the normalised inverse-distance weights
// w_i = (1/max(d_i, eps)) / sum_j (1/max(d_j, eps))  and 32-bit indices.
struct KnnFused {
  float eps;
  float *weight;
  int32_t *index32;
};

template <int K, int Q, bool FUSED = false>
__global__ void __launch_bounds__(KN_THREADS)
knn_small_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2,
                 float *__restrict__ dist, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl,
                 KnnFused fu = KnnFused()) {
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
      const int lim = (min(TILE, N2 - t0) + GK - 1) / GK * GK;
#pragma unroll 4
      for (int u0 = 0; u0 < lim; u0 += GK) {
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
        if constexpr (FUSED) {
          float inv[K], sum = 0.f;
#pragma unroll
          for (int c = 0; c < K; ++c) {
            inv[c] = __fdiv_rn(1.0f, fmaxf(kd[s][c], fu.eps));
            sum = c == 0 ? inv[0] : __fadd_rn(sum, inv[c]);
          }
          float *ow = fu.weight + (b * N1 + i) * K;
          int32_t *oi = fu.index32 + (b * N1 + i) * K;
#pragma unroll
          for (int c = 0; c < K; ++c) {
            ow[c] = __fdiv_rn(inv[c], sum);
            oi[c] = ki[s][c];
          }
        } else {
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
// Two-pass kernel for 4 < k <= 128 (fp32).
//
// Pass 1 sweeps all keys with the cheap filter value a (3 FMA per pair) and keeps, per query, the
// minimum of a over NCH >= 2k interleaved key classes (class = position inside a key tile divided by
// the keys per class, so every class is spread over the whole cloud whatever the key order).  The k-th smallest class
// minimum tau bounds the k-th smallest exact distance from above: the k classes below it each
// hold a distinct key with a <= tau, and for any key
//     d <= (a + 22.2u |r|^2 + 3.1u |q|^2 + |q|^2) (1 + 5.1u)
// (upper counterpart of the bound derived in sweep.cuh; |r|^2 <= the cloud's maximum).
// Pass 2 sweeps the keys again and records every key whose filter value admits d <= that bound --
// typically about 1.4 k candidates -- and the exact top-k by (distance, index) is then selected
// among the candidates only.  No data-dependent work happens inside the sweeps, so the lanes of a
// warp stay in step however the insert pattern of a one-pass top-k would look.
//
// Work split: a block of 4 warps serves 32*Q queries; warp s sweeps the s-th quarter of every key
// tile for all of them (lane = query), so a cloud of a few thousand queries still fills the GPU.
// Class minima are merged through shared memory.  Candidates of a query go to ONE list per query
// (slot claimed with a shared-memory atomic, so the four warps share the space and its order is
// arbitrary); the final selection ranks every candidate by (distance, index) against all others of
// its query, which is order independent, and writes it straight to its output position.
// Shared memory is laid out so that the exact candidate distances reuse the key tiles and class
// minima (dead by then): 30 KB per block for Q = 2, which keeps seven blocks (28 warps) per SM.
// If a list overflows (massive ties, adversarial or non-finite input) the query falls back to an
// exact insertion scan over all keys.
constexpr int KT_THREADS = 128;
constexpr int KT_SPLIT = KT_THREADS / 32;  // key quarters per tile
// KT_NCH key classes (32 to 256: at least two per wanted neighbour, i.e. k <= KT_NCH / 2; a warp
// holds the minima of its KT_NCH / 4 classes in registers) and KT_QCAP candidate slots per query
// (about 1.4 k candidates are expected) are template parameters of the kernel:
//     k <= 16: 32 classes, 56 slots, one or two queries per lane
//     k <= 32: 64 classes, 104 slots, one query per lane
//     k <= 64: 128 classes, 192 slots, one query per lane
//     k <= 128: 256 classes, 384 slots, one query per lane, 512-key tiles (KT_TILE; 256 otherwise)
template <int Q, int KT_NCH, int KT_QCAP, int KT_TILE>
constexpr size_t kt_smem_bytes() {
  return (size_t)2 * KT_TILE * 16 + (size_t)KT_NCH * 32 * Q * 4 + (size_t)KT_QCAP * 32 * Q * 4;
}

// Predicated append: if !(a >= thr), claim a slot of the query's list and store j there (when the
// slot exists).  Written in PTX so that it stays five straight-line instructions per pair.
template <int STRIDE_BYTES, int KT_QCAP>
__device__ __forceinline__ void kt_append(float a, float thr, unsigned cnt_addr, unsigned cand_addr, int j) {
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
      "f"(thr), "r"(cnt_addr), "r"(cand_addr), "r"(j), "n"(KT_QCAP), "n"(STRIDE_BYTES));
}

// Q = queries per lane (1 or 2): a block serves 32*Q queries.  Two queries per lane halve the
// shared-memory reads per pair, one keeps more blocks in flight when queries are few.
template <int Q, int KT_NCH, int KT_QCAP, int MINB, int KT_TILE>
__global__ void __launch_bounds__(KT_THREADS, MINB)
knn_twopass_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2, int k,
                   float *__restrict__ dist, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  constexpr int PER = KT_TILE / KT_THREADS;
  constexpr int CPW = KT_NCH / KT_SPLIT;          // classes per warp: 8, 16 or 32
  constexpr int PPC = KT_TILE / KT_SPLIT / CPW / 2;  // key pairs per class, tile and warp: 4, 2 or 1
  constexpr int QS = 32 * Q;              // query slots per block
  constexpr int NSUB = KT_THREADS / QS;   // threads per query in the selection
  extern __shared__ __align__(16) unsigned char kt_smem[];
  float4 *tile = reinterpret_cast<float4 *>(kt_smem);                                  // [2][KT_TILE], pair layout
  float *cm = reinterpret_cast<float *>(kt_smem + 2 * KT_TILE * 16);                   // [KT_NCH][QS] class minima
  int *cand = reinterpret_cast<int *>(kt_smem + 2 * KT_TILE * 16 + KT_NCH * QS * 4);   // [KT_QCAP][QS]
  float *cd = reinterpret_cast<float *>(kt_smem);  // [KT_QCAP][QS] exact distances; reuses tile + cm after pass 2
  static_assert(2 * KT_TILE * 16 + KT_NCH * QS * 4 >= KT_QCAP * QS * 4, "candidate distances fit into tile + cm");
  static_assert(KT_QCAP >= KT_NCH / 2, "the fallback keeps its k <= KT_NCH / 2 list in the query's own column");
  static_assert(PPC >= 1, "at least one key pair per class, tile and warp");
  __shared__ int ccnt[QS];
  __shared__ float s_rmax[KT_SPLIT];
  __shared__ float s_tau[QS];
  __shared__ float sq[3][QS];
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
    __syncthreads();  // the previous iteration's candidate distances alias the tile; sq is rewritten
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const int i = ibase + s * 32 + lane;
      valid[s] = i < N1;
      qx[s] = qy[s] = qz[s] = 0.f;
      if (valid[s]) load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx[s], qy[s], qz[s]);
      if (part == 0) {
        sq[0][s * 32 + lane] = qx[s];
        sq[1][s * 32 + lane] = qy[s];
        sq[2][s * 32 + lane] = qz[s];
      }
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

    // ---- pass 1: minima of the filter value over this warp's 8 classes
    float cmin[Q][CPW];
#pragma unroll
    for (int s = 0; s < Q; ++s)
#pragma unroll
      for (int c = 0; c < CPW; ++c) cmin[s][c] = pinf();
    fetch(0);
    commit(tile);
    __syncthreads();
    for (int t = 0; t < ntiles; ++t) {
      const float4 *tl = tile + (t & 1) * KT_TILE + part * (KT_TILE / KT_SPLIT);
      if (t + 1 < ntiles) fetch((t + 1) * KT_TILE);
#pragma unroll
      for (int c = 0; c < CPW; ++c) {
#pragma unroll
        for (int p = 0; p < PPC; ++p) {
          const float4 A = tl[c * 2 * PPC + 2 * p], Bv = tl[c * 2 * PPC + 2 * p + 1];
          const float2 kx = make_float2(A.x, A.y), ky = make_float2(A.z, A.w);
          const float2 kz = make_float2(Bv.x, Bv.y), kw = make_float2(Bv.z, Bv.w);
#pragma unroll
          for (int s = 0; s < Q; ++s) {
            const float2 a = __ffma2_rn(mx[s], kx, __ffma2_rn(my[s], ky, __ffma2_rn(mz[s], kz, kw)));
            cmin[s][c] = sweep_min3(cmin[s][c], a.x, a.y);
          }
        }
      }
      if (t + 1 < ntiles) commit(tile + ((t + 1) & 1) * KT_TILE);
      __syncthreads();
    }
#pragma unroll
    for (int s = 0; s < Q; ++s)
#pragma unroll
      for (int c = 0; c < CPW; ++c) cm[(part * CPW + c) * QS + s * 32 + lane] = cmin[s][c];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, o));
    if (lane == 0) s_rmax[part] = rmax;
    if (tid < QS) s_tau[tid] = pinf();
    __syncthreads();
    rmax = fmaxf(fmaxf(s_rmax[0], s_rmax[1]), fmaxf(s_rmax[2], s_rmax[3]));

    // k-th smallest class minimum of each query: rank by counting (ties broken by class number);
    // each warp ranks its own 8 classes and the one with rank k-1 publishes the value.
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
    // Upper bound of the k-th smallest exact distance (constants rounded up generously to cover
    // the roundings of this very computation), then the filter threshold that admits every key
    // at or below it.  Anything non-finite sends the query to the exact fallback: its counter
    // starts beyond the capacity and its threshold admits nothing.
    float thr[Q];
#pragma unroll
    for (int s = 0; s < Q; ++s) {
      const float tau = s_tau[s * 32 + lane];
      const float a_up = tau + 32.f * u * rmax + 8.f * u * qq[s];
      const float d_up = (a_up + qq[s] * (1.f + 8.f * u)) * (1.f + 10.f * u) + 1e-37f;
      const float lim = __int_as_float(__float_as_int(fmaxf(d_up, 0.f)) + 1);  // next float up
      const bool finite = d_up < 3.0e38f && rmax < 1.0e30f && qq[s] < 1.0e30f;
      thr[s] = (finite && valid[s]) ? sweep_threshold(lim, qq[s]) : -pinf();
      if (part == 0) ccnt[s * 32 + lane] = (finite || !valid[s]) ? 0 : KT_QCAP + 1;
    }

    // ---- pass 2: collect the candidates (padding keys carry w = +inf and never pass)
    fetch(0);
    commit(tile);
    __syncthreads();
    for (int t = 0; t < ntiles; ++t) {
      const int t0 = t * KT_TILE + part * (KT_TILE / KT_SPLIT);
      const float4 *tl = tile + (t & 1) * KT_TILE + part * (KT_TILE / KT_SPLIT);
      if (t + 1 < ntiles) fetch((t + 1) * KT_TILE);
#pragma unroll 2
      for (int u0 = 0; u0 < KT_TILE / KT_SPLIT; u0 += 4) {
        // Two key pairs (four keys) at a time: one minimum and one compare per query decide
        // whether any of its four filter values passes; only then are the four appends executed
        // (about 2 % of the lanes, half of the warps).
        float2 a[2][Q];
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          const float4 A = tl[u0 + 2 * p], Bv = tl[u0 + 2 * p + 1];
          const float2 kx = make_float2(A.x, A.y), ky = make_float2(A.z, A.w);
          const float2 kz = make_float2(Bv.x, Bv.y), kw = make_float2(Bv.z, Bv.w);
#pragma unroll
          for (int s = 0; s < Q; ++s)
            a[p][s] = __ffma2_rn(mx[s], kx, __ffma2_rn(my[s], ky, __ffma2_rn(mz[s], kz, kw)));
        }
        const int j = t0 + u0;
#pragma unroll
        for (int s = 0; s < Q; ++s) {
          const float m = fminf(sweep_min3(a[0][s].x, a[0][s].y, a[1][s].x), a[1][s].y);
          if (m < thr[s]) {
            const unsigned ca = cnt_base + 4u * (s * 32 + lane), da = cand_base + 4u * (s * 32 + lane);
            kt_append<QS * 4, KT_QCAP>(a[0][s].x, thr[s], ca, da, j);
            kt_append<QS * 4, KT_QCAP>(a[0][s].y, thr[s], ca, da, j + 1);
            kt_append<QS * 4, KT_QCAP>(a[1][s].x, thr[s], ca, da, j + 2);
            kt_append<QS * 4, KT_QCAP>(a[1][s].y, thr[s], ca, da, j + 3);
          }
        }
      }
      if (t + 1 < ntiles) commit(tile + ((t + 1) & 1) * KT_TILE);
      __syncthreads();
    }

    // ---- exact selection: NSUB threads per query.  First the exact distance of every candidate,
    // then each candidate's rank by (distance, index) among its query's candidates; ranks below k
    // go straight to the output row.
    const int col = tid % QS, sub = tid / QS;
    const int iq = ibase + col;
    const bool qvalid = iq < N1;
    const int n = ccnt[col];
    const float cqx = sq[0][col], cqy = sq[1][col], cqz = sq[2][col];
    // A list that overflowed, or -- which the bound derivation rules out for finite input, but which
    // costs nothing to guard -- holds fewer than k candidates, sends its query to the exact scan.
    const bool listed = n >= k && n <= KT_QCAP;
    if (qvalid && listed) {
      for (int c = sub; c < n; c += NSUB) {
        const int j = cand[c * QS + col];
        float rx, ry, rz;
        load_xyz(rb, j, kl, rx, ry, rz);
        cd[c * QS + col] = sqdist<float>(rx, ry, rz, cqx, cqy, cqz);
      }
    }
    __syncthreads();
    if (qvalid) {
      float *od = dist + (b * N1 + iq) * (int64_t)k;
      const int64_t orow = (b * N1 + iq) * (int64_t)k;
      if (listed) {
        for (int c = sub; c < n; c += NSUB) {
          const float d = cd[c * QS + col];
          const int j = cand[c * QS + col];
          int rank = 0;
          for (int o = 0; o < n; ++o) {
            const float w = cd[o * QS + col];
            const int jo = cand[o * QS + col];
            rank += (w < d || (w == d && jo < j)) ? 1 : 0;
          }
          if (rank < k) {
            od[rank] = d;
            index.put(orow + rank, j);
          }
        }
      } else if (sub == 0) {
        // Exact insertion scan; the sorted list lives in the first k slots of this query's own
        // column of cd / cand (nobody else touches the column of an overflowed query).
        int nk = 0;
        for (int j = 0; j < N2; ++j) {
          float rx, ry, rz;
          load_xyz(rb, j, kl, rx, ry, rz);
          const float d = sqdist<float>(rx, ry, rz, cqx, cqy, cqz);
          if (nk == k) {
            const float dl = cd[(k - 1) * QS + col];
            if (!(d < dl || (d == dl && j < cand[(k - 1) * QS + col]))) continue;
          }
          int pos = nk < k ? nk : k - 1;
          while (pos > 0) {
            const float dp = cd[(pos - 1) * QS + col];
            if (!(d < dp || (d == dp && j < cand[(pos - 1) * QS + col]))) break;
            cd[pos * QS + col] = dp;
            cand[pos * QS + col] = cand[(pos - 1) * QS + col];
            --pos;
          }
          cd[pos * QS + col] = d;
          cand[pos * QS + col] = j;
          if (nk < k) ++nk;
        }
        for (int c = 0; c < k; ++c) {
          od[c] = cd[c * QS + col];
          index.put(orow + c, cand[c * QS + col]);
        }
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

template <int K, int Q>
int knn_small(const float *query, const float *key, int64_t B, int N1, int N2, float *dist, const KnnIo &io,
              cudaStream_t st) {
  const int64_t per = KN_THREADS * Q;
  const int64_t total = B * ((N1 + per - 1) / per);
  const int64_t cap = (int64_t)sm_count() * 256;
  knn_small_kernel<K, Q><<<(unsigned)(total < cap ? total : cap), KN_THREADS, 0, st>>>(query, key, B, N1, N2, dist,
                                                                                      io.index, total, io.ql, io.kl);
  return check_launch("knn_small_kernel");
}

template <int K>
int knn_small_q(const float *query, const float *key, int64_t B, int N1, int N2, float *dist, const KnnIo &io,
                cudaStream_t st) {
  const int64_t sms = sm_count();
  if (B * (int64_t)N1 >= sms * 2 * KN_THREADS * 2) return knn_small<K, 2>(query, key, B, N1, N2, dist, io, st);
  return knn_small<K, 1>(query, key, B, N1, N2, dist, io, st);
}

template <int Q>
int three_nn_fused_q(const float *query, const float *key, int64_t B, int N1, int N2, const KnnFused &fu,
                     XyzLayout ql, XyzLayout kl, cudaStream_t st) {
  const int64_t per = KN_THREADS * Q;
  const int64_t total = B * ((N1 + per - 1) / per);
  const int64_t cap = (int64_t)sm_count() * 256;
  knn_small_kernel<3, Q, true><<<(unsigned)(total < cap ? total : cap), KN_THREADS, 0, st>>>(
      query, key, B, N1, N2, nullptr, index_out(nullptr, 0), total, ql, kl, fu);
  return check_launch("knn_small_kernel (fused weights)");
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

// Three nearest keys of every query with inverse-distance weights (see KnnFused); N2 >= 3.
int three_nn_fused_f32(const float *query, const float *key, int64_t B, int64_t N1, int64_t N2, int channel_first,
                       float eps, float *weight, int32_t *index32, cudaStream_t st) {
  if (B * N1 == 0) return TK3D_OK;
  KnnFused fu;
  fu.eps = eps;
  fu.weight = weight;
  fu.index32 = index32;
  const XyzLayout ql = xyz_layout(channel_first, N1), kl = xyz_layout(channel_first, N2);
  if (B * N1 >= (int64_t)sm_count() * 2 * KN_THREADS * 2)
    return three_nn_fused_q<2>(query, key, B, (int)N1, (int)N2, fu, ql, kl, st);
  return three_nn_fused_q<1>(query, key, B, (int)N1, (int)N2, fu, ql, kl, st);
}

}  // namespace tk3d

namespace tk3d {
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
  io.index = index_out(index, index32);
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
  // counts below) and a few keys in every class: N2 >= 4 k, at least 256 (512 for k > 64).
  if (k <= 128 && N2 >= 4 * k && N2 >= (k > 64 ? 512 : 256)) {
    if (k <= 16) {
      if (B * N1 >= (int64_t)sm_count() * 4 * 64)
        return knn_twopass<2, 32, 56, 7>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
      return knn_twopass<1, 32, 56, 7>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
    }
    if (k <= 32) return knn_twopass<1, 64, 104, 5>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
    if (k <= 64) return knn_twopass<1, 128, 192, 4>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
    return knn_twopass<1, 256, 384, 2, 512>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
  }
  if (k <= 128) {
    const int64_t sms = sm_count();
    if (k <= 32 && B * N1 >= sms * 2 * KN_THREADS * 2)
      return knn_buffered<2>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
    return knn_buffered<1>(q, r, B, (int)N1, (int)N2, (int)k, d, io, st);
  }
  return knn_generic<float>(q, r, B, N1, N2, k, d, io, st);
}

extern "C" int tk3d_knn(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, int64_t k,
                        void *distance, int64_t *index, int dtype, void *stream) {
  return knn_impl(query, key, B, N1, N2, k, 0, distance, index, 0, dtype, stream);
}

extern "C" int tk3d_knn_layout(const void *query, const void *key, int64_t B, int64_t N1, int64_t N2, int64_t k,
                               int xyz_channel_first, void *distance, void *index, int index_dtype, int dtype,
                               void *stream) {
  TK3D_REQUIRE(index_dtype == TK3D_I64 || index_dtype == TK3D_I32, TK3D_ERR_DTYPE, "knn: index_dtype %d", index_dtype);
  return knn_impl(query, key, B, N1, N2, k, xyz_channel_first != 0, distance, index, index_dtype == TK3D_I32, dtype,
                  stream);
}
