// Brute-force KNN for large k (float32, 32 < k <= 256): selection by radix instead of by insertion.
//
// Keeping the k best of a query in a list or heap costs an insertion per accepted key, and with one
// query per lane every insertion stalls the other 31 lanes of its warp: for k = 200 on 4096 keys the
// heap kernel spends nearly all of its time there.  Here nothing data dependent happens inside the
// key sweeps.  A block of eight warps serves 32 queries (lane = query; every warp sweeps an eighth of
// each 256-key tile) and finds the k-th smallest distance of each query EXACTLY by a most-significant-
// digit radix selection on the bit pattern of the distance (non-negative floats order like their
// bits): one sweep per byte, each counting the keys whose higher bytes equal the digits found
// so far into a 256-bin histogram per query in shared memory ([bin][lane]: a lane only ever touches
// its own bank).  Usually two bytes are enough: when the keys up to and including the 16-bit bucket
// of the k-th distance fit the list of every query of the block, one more sweep collects them and
// the sort finishes the selection.  Otherwise (massive ties) all four bytes are resolved and a
// fifth sweep collects the keys below that distance (in any order) and, by the
// position scheme of the ball query (hits of a slice as a bit mask, counts exchanged at the tile
// barrier), the first keys in index order AT that distance, exactly k in all; a bitonic network
// over (distance bits, index) as one 64-bit word, run by the eight warps together on the lists in
// shared memory, puts them in the (distance, index) order every other path emits.
//
// Three to five sweeps of the plain distance (two keys per packed FP32 instruction) are far from the
// FP32 roofline, but they cost nearly the same for every k and every key order: 4 x 4096 x 4096 with
// k = 200 takes a fraction of a millisecond where the heap kernel took 10.8 ms (the reference's
// bounded-set kernel, torkit3d/csrc/cuda/knn_distance_kernel.cu:102-177 with
// torkit3d/csrc/include/mink.cuh:61-89, 8.6 ms).  A NaN distance (a NaN coordinate) is given the
// canonical NaN pattern, which is above +inf as an integer, so such keys order last, by index.
#include <limits.h>

#include "tk3d_common.cuh"

namespace tk3d {
namespace {

constexpr int SEL_THREADS = 256;
constexpr int SEL_SPLIT = SEL_THREADS / 32;
constexpr int SEL_TILE = 256;
constexpr int SEL_QK = SEL_TILE / SEL_SPLIT;  // keys per warp per tile: one 64-bit mask
constexpr int SEL_BINS = 256;

__device__ __forceinline__ unsigned sel_bits(float d) {
  return d == d ? __float_as_uint(d) : 0x7fc00000u;  // d >= +0 or NaN
}

// smem: [hist 256 x 32 ints | list n2 x 32 u64] (the list aliases the histogram) + tiles
__global__ void __launch_bounds__(SEL_THREADS)
knn_select_kernel(const float *__restrict__ query, const float *__restrict__ key, int64_t B, int N1, int N2, int k, int n2,
                  float *__restrict__ dist, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl, float one) {
  extern __shared__ __align__(16) unsigned char sel_smem[];
  int *hist = reinterpret_cast<int *>(sel_smem);                                // [256][32]
  unsigned long long *list = reinterpret_cast<unsigned long long *>(sel_smem);  // [n2][32], after the histograms
  __shared__ float4 tile[2][SEL_TILE];  // key pair p: [2p] = (x0, x1, y0, y1), [2p+1] = (z0, z1, -, -)
  __shared__ int tcount[2][SEL_SPLIT][32];
  __shared__ int psum[SEL_SPLIT][32];
  __shared__ int cless[32];
  const int tid = threadIdx.x, lane = tid & 31, part = tid >> 5;
  const int chunks = (N1 + 31) / 32;
  const int ntiles = (N2 + SEL_TILE - 1) / SEL_TILE;

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int i = (int)(blk % chunks) * 32 + lane;
    const bool valid = i < N1;
    float qx = 0.f, qy = 0.f, qz = 0.f;
    if (valid) load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx, qy, qz);
    const float *rb = key + b * (int64_t)N2 * 3;
    // The distance of TWO keys per instruction on the packed FP32 pipe: key - query as key + (-query),
    // packed squares, and the two sums as fma(x, one, y) with `one` = 1.0f from a kernel argument --
    // round(x * 1 + y) = round(x + y), and a multiplier the compiler cannot see keeps it from fusing
    // the squares into the sums (see the note in fps.cu).  Bit for bit ((dx*dx + dy*dy) + dz*dz).
    const float2 nqx = make_float2(-qx, -qx), nqy = make_float2(-qy, -qy), nqz = make_float2(-qz, -qz);
    const float2 one2 = make_float2(one, one);

    // One sweep over the keys: tiles are staged by the whole block (next tile fetched into
    // registers while the current one is used), `body(u, j, bits)` sees every key of this warp's
    // slices: position in the slice, index in the cloud, bit pattern of its distance.
    auto sweep = [&](auto &&body, auto &&tile_end) {
      float4 nxt[SEL_TILE / SEL_THREADS];
      auto fetch = [&](int t0) {
#pragma unroll
        for (int p = 0; p < SEL_TILE / SEL_THREADS; ++p) {
          const int j = t0 + tid + p * SEL_THREADS;
          float x = 0.f, y = 0.f, z = 0.f;
          if (j < N2) load_xyz(rb, j, kl, x, y, z);
          nxt[p] = make_float4(x, y, z, 0.f);
        }
      };
      auto commit = [&](float4 *dst) {
#pragma unroll
        for (int p = 0; p < SEL_TILE / SEL_THREADS; ++p) {
          const int u = tid + p * SEL_THREADS;
          float *f = reinterpret_cast<float *>(dst) + (u >> 1) * 8 + (u & 1);
          f[0] = nxt[p].x;
          f[2] = nxt[p].y;
          f[4] = nxt[p].z;
        }
      };
      fetch(0);
      commit(tile[0]);
      __syncthreads();
      for (int t = 0; t < ntiles; ++t) {
        const int t0 = t * SEL_TILE + part * SEL_QK;
        const float4 *tl = tile[t & 1] + part * SEL_QK;
        if (t + 1 < ntiles) fetch((t + 1) * SEL_TILE);
        const int lim = min(SEL_QK, N2 - t0);  // <= 0 for slices beyond the cloud
#pragma unroll 4
        for (int u = 0; u < lim; u += 2) {
          const float4 A = tl[u];
          const float2 kz = *reinterpret_cast<const float2 *>(tl + u + 1);
          const float2 dx = __fadd2_rn(make_float2(A.x, A.y), nqx), dy = __fadd2_rn(make_float2(A.z, A.w), nqy);
          const float2 dz = __fadd2_rn(kz, nqz);
          const float2 d =
              __ffma2_rn(__ffma2_rn(__fmul2_rn(dx, dx), one2, __fmul2_rn(dy, dy)), one2, __fmul2_rn(dz, dz));
          body(u, t0 + u, sel_bits(d.x));
          if (u + 1 < lim) body(u + 1, t0 + u + 1, sel_bits(d.y));
        }
        if (t + 1 < ntiles) commit(tile[(t + 1) & 1]);
        tile_end(t, t0);
      }
    };

    // ---- the k-th smallest distance, one byte per sweep
    unsigned prefix = 0;  // digits found so far (the high bytes of the k-th distance)
    bool short_cut = false;
    int krem = k;         // rank of the k-th distance among the keys that share those digits
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int e = tid; e < SEL_BINS * 32; e += SEL_THREADS) hist[e] = 0;
      __syncthreads();
      sweep(
          [&](int, int, unsigned bits) {
            const bool match = pass == 0 || (bits >> (shift + 8)) == prefix;
            if (match) atomicAdd(&hist[((bits >> shift) & 255u) * 32 + lane], 1);
          },
          [&](int, int) { __syncthreads(); });
      // which bin holds the krem-th key: every warp adds up a share of the bins, then all warps
      // walk the share that holds it (the same result in every warp, lane = query)
      int s = 0;
      constexpr int QB = SEL_BINS / SEL_SPLIT;  // bins per warp
      for (int bin = part * QB; bin < part * QB + QB; ++bin) s += hist[bin * 32 + lane];
      psum[part][lane] = s;
      __syncthreads();
      int before = 0, quarter = 0;
#pragma unroll
      for (int w = 0; w < SEL_SPLIT; ++w) {
        const int c = psum[w][lane];
        if (quarter == w && before + c < krem && w + 1 < SEL_SPLIT) {
          before += c;
          quarter = w + 1;
        }
      }
      int bin = quarter * QB;
      int cbin = hist[bin * 32 + lane];
      for (int step = 0; step < QB - 1 && before + cbin < krem; ++step) {
        before += cbin;
        ++bin;
        cbin = hist[bin * 32 + lane];
      }
      prefix = (prefix << 8) | (unsigned)bin;
      krem -= before;
      // After two bytes the bucket of the k-th distance usually holds a handful of keys: if, for
      // every query of the block, the keys up to and including that bucket fit the list, they are
      // collected as they are and the sort below does the rest -- three sweeps instead of five.
      // (The vote is also the barrier after which the histogram may be cleared or reused.)
      const bool fits = pass == 1 && (k - krem) + cbin <= n2;
      if (__syncthreads_and(fits)) {
        short_cut = true;
        break;
      }
    }
    if (part == 0) cless[lane] = 0;
    if (short_cut) {
      // ---- collect every key whose two high bytes do not exceed those of the k-th distance
      for (int e = tid; e < n2 * 32; e += SEL_THREADS) list[e] = ~0ull;  // unused slots sort last
      __syncthreads();
      sweep(
          [&](int, int j, unsigned bits) {
            if ((bits >> 16) <= prefix) {
              const int slot = atomicAdd(&cless[lane], 1);  // at most n2 keys, by the vote above
              list[slot * 32 + lane] = ((unsigned long long)bits << 32) | (unsigned)j;
            }
          },
          [&](int, int) { __syncthreads(); });
    } else {
    const unsigned kth = prefix;  // bit pattern of the k-th smallest distance
    const int need_eq = krem;     // keys AT that distance that belong to the result (>= 1)
    const int nless = k - need_eq;

    // ---- collect: everything below kth, and the first need_eq keys (by index) at kth
    for (int e = k * 32 + tid; e < n2 * 32; e += SEL_THREADS) list[e] = ~0ull;  // padding sorts last
    __syncthreads();
    unsigned long long mask = 0;
    int cnt = 0, eq_done = 0;
    sweep(
        [&](int u, int j, unsigned bits) {
          if (bits < kth) {
            const int slot = atomicAdd(&cless[lane], 1);  // exactly nless keys take this branch
            list[slot * 32 + lane] = ((unsigned long long)bits << 32) | (unsigned)j;
          }
          if (bits == kth) {
            mask |= 1ull << u;
            ++cnt;
          }
        },
        [&](int t, int t0) {
          tcount[t & 1][part][lane] = cnt;
          __syncthreads();
          int before = 0, total = 0;
#pragma unroll
          for (int w = 0; w < SEL_SPLIT; ++w) {
            const int c = tcount[t & 1][w][lane];
            if (w < part) before += c;
            total += c;
          }
          int pos = eq_done + before;
          while (mask != 0 && pos < need_eq) {
            const int bit = __ffsll((long long)mask) - 1;
            mask &= mask - 1;
            list[(nless + pos) * 32 + lane] = ((unsigned long long)kth << 32) | (unsigned)(t0 + bit);
            ++pos;
          }
          eq_done += total;
          mask = 0;
          cnt = 0;
        });
    }
    __syncthreads();

    // ---- sort the n2 (k rounded up to a power of two, padded with all-ones) entries of every list
    // by (distance bits, index): the pairs of each compare-exchange step are dealt to the warps
    for (int size = 2; size <= n2; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int p = part; p < (n2 >> 1); p += SEL_SPLIT) {
          const int lo = ((p & ~(stride - 1)) << 1) | (p & (stride - 1));
          const int hi = lo | stride;
          const bool up = (lo & size) == 0;
          const unsigned long long a = list[lo * 32 + lane], c = list[hi * 32 + lane];
          if ((a > c) == up) {
            list[lo * 32 + lane] = c;
            list[hi * 32 + lane] = a;
          }
        }
        __syncthreads();
      }
    }
    if (valid) {
      const int64_t row = (b * N1 + i) * (int64_t)k;
      for (int sl = part; sl < k; sl += SEL_SPLIT) {
        const unsigned long long e = list[sl * 32 + lane];
        dist[row + sl] = __uint_as_float((unsigned)(e >> 32));
        index.put(row + sl, (int64_t)(unsigned)(e & 0xffffffffu));
      }
    }
    __syncthreads();  // the lists become histograms again
  }
}

size_t select_smem(int n2) {
  const size_t h = (size_t)SEL_BINS * 32 * sizeof(int), l = (size_t)n2 * 32 * sizeof(unsigned long long);
  return h > l ? h : l;
}

}  // namespace

// k-nearest keys by radix selection; the caller has checked 1 <= k <= 256, k <= N2 < 2^31.
int knn_select_f32(const float *query, const float *key, int64_t B, int N1, int N2, int k, float *dist, IndexOut index,
                   XyzLayout ql, XyzLayout kl, cudaStream_t st) {
  // list length: a power of two with some room above k for the keys that share the 16-bit bucket
  // of the k-th distance (the short cut of the kernel), at most 256
  int n2 = 2;
  while (n2 < k + 8 && n2 < 256) n2 <<= 1;
  while (n2 < k) n2 <<= 1;
  const size_t smem = select_smem(n2);
  if (smem + 12 * 1024 > 48 * 1024) TK3D_CUDA(raise_smem_limit((const void *)knn_select_kernel, (int)smem));
  const int64_t total = B * ((N1 + 31) / 32);
  const int64_t cap = (int64_t)sm_count() * 32;
  knn_select_kernel<<<(unsigned)(total < cap ? total : cap), SEL_THREADS, smem, st>>>(query, key, B, N1, N2, k, n2, dist,
                                                                                    index, total, ql, kl, 1.0f);
  return check_launch("knn_select_kernel");
}

}  // namespace tk3d

TK3D_BOUNDS_TU(knn_select)
