// Brute-force k nearest neighbours in a C-dimensional feature space (DGCNN's dynamic graph:
// torkit3d/models/classification/dgcnn.py:58-61 calls torkit3d/ops/native.py:4-30, cdist + topk,
// on [B, C, N] features).
//
// Squared distance of a (query, key) pair: acc = 0; for c = 0 .. C-1: acc = fma(d_c, d_c, acc) with
// d_c = key_c - query_c -- one rounding per channel, summed in channel order, which a CPU loop with
// fmaf() reproduces bit for bit.  (The reference's cdist goes through a matrix product and is
// itself only accurate to about 1e-6 of |q|^2 + |r|^2; this form is cheaper than it looks -- two
// FP32 instructions per pair and channel -- and needs no tensor cores at DGCNN's sizes: 32 clouds
// of 1024 points with 64 channels are 4.3 GFLOP.)
//
// A block of 8 warps owns 32 queries; warp w owns queries 4w .. 4w+3 and, for every tile of 128
// keys, lane l holds the 4 x 4 distances of those queries to keys l, l+32, l+64, l+96 in registers
// (channel slices of 16 are staged in shared memory: one broadcast LDS.128 for the queries and
// four conflict-free LDS.32 for the keys feed 16 subtractions and 16 FMAs).  The same warp then
// selects: each query's k best so far form a list sorted by (distance, index) that is spread over
// the warp's registers (entry m lives in lane m % 32, slot m / 32); candidates that order before
// the k-th entry are found with a ballot and inserted one at a time with a rank count (ballot +
// popc) and a one-lane shift (shfl_up).  Ties go to the lower index; rows come out sorted.
#include <limits.h>

#include "tk3d_common.cuh"

namespace tk3d {
namespace {

constexpr int FK_THREADS = 256;
constexpr int FK_QT = 32;   // queries per block
constexpr int FK_KT = 128;  // keys per tile
constexpr int FK_CS = 16;   // channels per slice
constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ bool before(float d, int i, float e, int j) { return d < e || (d == e && i < j); }

// KS: list slots per lane (capacity 32 * KS >= k).  CF: channel-first tensors [B, C, N], otherwise
// point-major [B, N, C].
template <int KS, bool CF>
__global__ void __launch_bounds__(FK_THREADS, KS <= 2 ? 3 : 2)
feature_knn_kernel(const float *__restrict__ query, const float *__restrict__ key, int C, int N1, int N2, int k,
                   float *__restrict__ dist, int64_t *__restrict__ index, int64_t blocks_total) {
  __shared__ __align__(16) float qs[FK_CS][FK_QT];
  __shared__ float ks[FK_CS][FK_KT + 1];  // + 1: the point-major staging stores spread over the banks
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunks = (N1 + FK_QT - 1) / FK_QT;
  const float pinf = __int_as_float(0x7f800000);
  const int kslot = (k - 1) >> 5, klane = (k - 1) & 31;

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int q0 = (int)(blk % chunks) * FK_QT;
    const float *qb = query + b * (int64_t)C * N1;
    const float *kb = key + b * (int64_t)C * N2;

    float ld[4][KS], thd[4];
    int li[4][KS], thi[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      thd[a] = pinf;
      thi[a] = INT_MAX;
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        ld[a][s] = pinf;
        li[a][s] = INT_MAX;  // sentinel: orders after every real (distance, index)
      }
    }

    for (int j0 = 0; j0 < N2; j0 += FK_KT) {
      float acc[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) acc[a][bb] = 0.f;

      for (int c0 = 0; c0 < C; c0 += FK_CS) {
        __syncthreads();  // the previous slice has been consumed
#pragma unroll
        for (int r = 0; r < FK_CS * FK_QT / FK_THREADS; ++r) {
          const int e = tid + r * FK_THREADS;
          const int c = CF ? e / FK_QT : e % FK_CS, i = CF ? e % FK_QT : e / FK_CS;
          float v = 0.f;  // channels past C and queries past N1 read as zero on both sides
          if (c0 + c < C && q0 + i < N1)
            v = CF ? qb[(int64_t)(c0 + c) * N1 + q0 + i] : qb[(int64_t)(q0 + i) * C + c0 + c];
          qs[c][i] = v;
        }
#pragma unroll
        for (int r = 0; r < FK_CS * FK_KT / FK_THREADS; ++r) {
          const int e = tid + r * FK_THREADS;
          const int c = CF ? e / FK_KT : e % FK_CS, j = CF ? e % FK_KT : e / FK_CS;
          float v = 0.f;
          if (c0 + c < C && j0 + j < N2)
            v = CF ? kb[(int64_t)(c0 + c) * N2 + j0 + j] : kb[(int64_t)(j0 + j) * C + c0 + c];
          ks[c][j] = v;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < FK_CS; ++c) {
          const float4 qv = *reinterpret_cast<const float4 *>(&qs[c][4 * warp]);
          const float q[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
          for (int bb = 0; bb < 4; ++bb) {
            const float kv = ks[c][lane + 32 * bb];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
              const float df = __fsub_rn(kv, q[a]);
              acc[a][bb] = __fmaf_rn(df, df, acc[a][bb]);
            }
          }
        }
      }

      // Selection: this warp's four queries against the 128 keys of the tile.
#pragma unroll
      for (int a = 0; a < 4; ++a) {
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) {
          const int j = j0 + lane + 32 * bb;
          const float d = j < N2 ? acc[a][bb] : pinf;
          const int id = j < N2 ? j : INT_MAX;
          unsigned mask = __ballot_sync(FULL, before(d, id, thd[a], thi[a]));
          while (mask) {
            const int src = __ffs(mask) - 1;
            mask &= mask - 1;
            const float cd = __shfl_sync(FULL, d, src);
            const int ci = __shfl_sync(FULL, id, src);
            if (!before(cd, ci, thd[a], thi[a])) continue;  // the k-th entry moved since the ballot
            int pos = 0;                                     // entries that order before the candidate
#pragma unroll
            for (int s = 0; s < KS; ++s) pos += __popc(__ballot_sync(FULL, before(ld[a][s], li[a][s], cd, ci)));
#pragma unroll
            for (int s = KS - 1; s >= 0; --s) {  // top slot first: lower slots still hold the old entries
              float ud = __shfl_up_sync(FULL, ld[a][s], 1);
              int ui = __shfl_up_sync(FULL, li[a][s], 1);
              if (s > 0) {
                const float wd = __shfl_sync(FULL, ld[a][s - 1], 31);
                const int wi = __shfl_sync(FULL, li[a][s - 1], 31);
                if (lane == 0) ud = wd, ui = wi;
              }
              const int m = lane + 32 * s;
              if (m == pos) ld[a][s] = cd, li[a][s] = ci;
              else if (m > pos) ld[a][s] = ud, li[a][s] = ui;
            }
            float td = ld[a][0];
            int ti = li[a][0];
#pragma unroll
            for (int s = 1; s < KS; ++s)
              if (s == kslot) td = ld[a][s], ti = li[a][s];
            thd[a] = __shfl_sync(FULL, td, klane);
            thi[a] = __shfl_sync(FULL, ti, klane);
          }
        }
      }
    }

#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int qi = q0 + 4 * warp + a;
      if (qi < N1) {
        float *od = dist + (b * N1 + qi) * (int64_t)k;
        int64_t *oi = index + (b * N1 + qi) * (int64_t)k;
#pragma unroll
        for (int s = 0; s < KS; ++s) {
          const int m = lane + 32 * s;
          if (m < k) {
            od[m] = ld[a][s];
            oi[m] = li[a][s] == INT_MAX ? (int64_t)-1 : (int64_t)li[a][s];  // only with NaN inputs
          }
        }
      }
    }
  }
}

template <int KS>
int launch(const float *query, const float *key, int64_t B, int C, int N1, int N2, int k, bool cf, float *dist,
           int64_t *index, cudaStream_t st) {
  const int64_t total = B * ((N1 + FK_QT - 1) / FK_QT);
  const int64_t cap = (int64_t)sm_count() * 32;
  const unsigned grid = (unsigned)(total < cap ? total : cap);
  if (cf)
    feature_knn_kernel<KS, true><<<grid, FK_THREADS, 0, st>>>(query, key, C, N1, N2, k, dist, index, total);
  else
    feature_knn_kernel<KS, false><<<grid, FK_THREADS, 0, st>>>(query, key, C, N1, N2, k, dist, index, total);
  return check_launch("feature_knn_kernel");
}

}  // namespace
}  // namespace tk3d

using namespace tk3d;

extern "C" int tk3d_feature_knn(const void *query, const void *key, int64_t B, int64_t C, int64_t N1, int64_t N2,
                                int64_t k, int channel_first, void *dist, int64_t *index, int dtype, void *stream) {
  TK3D_RANGE("tk3d_feature_knn");
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "feature_knn: dtype %d", dtype);
  TK3D_REQUIRE(dtype == TK3D_F32, TK3D_ERR_UNSUPPORTED, "feature_knn: float32 only");
  TK3D_REQUIRE(B >= 0 && N1 >= 0 && N2 >= 0 && C >= 1, TK3D_ERR_SHAPE,
               "feature_knn: bad size (B=%lld C=%lld N1=%lld N2=%lld)", (long long)B, (long long)C, (long long)N1,
               (long long)N2);
  TK3D_REQUIRE(N1 < (1LL << 30) && N2 < (1LL << 30) && C < (1LL << 20), TK3D_ERR_SHAPE,
               "feature_knn: clouds limited to 2^30 points and 2^20 channels");
  TK3D_REQUIRE(k >= 1 && k <= N2, TK3D_ERR_K, "feature_knn: need 1 <= k <= N2 (k=%lld, N2=%lld)", (long long)k,
               (long long)N2);
  TK3D_REQUIRE(k <= 128, TK3D_ERR_UNSUPPORTED, "feature_knn: k up to 128 (got %lld)", (long long)k);
  if (B * N1 == 0) return TK3D_OK;
  TK3D_REQUIRE(query && key && dist && index, TK3D_ERR_NULL, "feature_knn: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  const float *q = (const float *)query, *r = (const float *)key;
  const bool cf = channel_first != 0;
  if (k <= 32) return launch<1>(q, r, B, (int)C, (int)N1, (int)N2, (int)k, cf, (float *)dist, index, st);
  if (k <= 64) return launch<2>(q, r, B, (int)C, (int)N1, (int)N2, (int)k, cf, (float *)dist, index, st);
  return launch<4>(q, r, B, (int)C, (int)N1, (int)N2, (int)k, cf, (float *)dist, index, st);
}

TK3D_BOUNDS_TU(feature_knn)
