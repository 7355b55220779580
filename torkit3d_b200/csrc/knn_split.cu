// Brute-force KNN for float64 clouds with few queries (and small k): the generic kernel of knn.cu
// gives every query one thread, which leaves a B200 nearly empty when there are only some ten
// thousand queries (8 clouds of 2048 points are 512 warps for 148 SMs).  Here a block serves 32
// queries with S warps: lane = query, warp s scans the s-th contiguous segment of the key cloud
// and keeps that segment's k best as a binary max-heap by (distance, index) in shared memory
// (replace the root and sift down, O(log k) per accepted key), heap-sorted at the segment's end;
// warp 0 then merges the S sorted lists of every query.  Segments are contiguous index ranges in
// ascending order, so taking the smaller head with a strict "<" (lower segment first on equal
// distances) reproduces the (distance, index) order of a single scan.
//
// Arithmetic and acceptance rule are those of the generic kernel and of the reference's loop
// (torkit3d/csrc/cuda/knn_distance_kernel.cu:65-82 with the bounded set of
// torkit3d/csrc/include/mink.cuh:61-89): exactly rounded ((dx*dx + dy*dy) + dz*dz), a key enters
// while the list is not full or when its distance is strictly below the current k-th.
#include <limits.h>

#include "tk3d_common.cuh"

namespace tk3d {
namespace {

constexpr int KS_STAGE = 64;  // keys a warp stages at a time

template <typename T>
__global__ void __launch_bounds__(256)
knn_split_kernel(const T *__restrict__ query, const T *__restrict__ key, int64_t B, int N1, int N2, int k, int S,
                 T *__restrict__ dist, IndexOut index, int64_t blocks_total, XyzLayout ql, XyzLayout kl) {
  extern __shared__ __align__(16) unsigned char ks_smem[];
  const int threads = 32 * S;
  T *ld = reinterpret_cast<T *>(ks_smem);                                  // [k][threads]
  T *stage = ld + (size_t)k * threads;                                     // [S][KS_STAGE][3]
  int *li = reinterpret_cast<int *>(stage + (size_t)S * KS_STAGE * 3);     // [k][threads]
  int *lcnt = li + (size_t)k * threads;                                    // [threads]
  const int tid = threadIdx.x, lane = tid & 31, seg = tid >> 5;
  const int chunks = (N1 + 31) / 32;
  const int seglen = (N2 + S - 1) / S;
  T *mystage = stage + (size_t)seg * KS_STAGE * 3;

  for (int64_t blk = blockIdx.x; blk < blocks_total; blk += gridDim.x) {
    const int64_t b = blk / chunks;
    const int i = (int)(blk % chunks) * 32 + lane;
    const bool valid = i < N1;
    T qx = 0, qy = 0, qz = 0;
    if (valid) load_xyz(query + b * 3 * (int64_t)N1, i, ql, qx, qy, qz);
    const T *rb = key + b * (int64_t)N2 * 3;
    const int j_begin = min(N2, seg * seglen), j_end = min(N2, j_begin + seglen);
    int cnt = 0;
    bool heaped = false;
    T worst = Exact<T>::inf();  // distance at the root once the heap is built
    auto D = [&](int p) -> T & { return ld[(size_t)p * threads + tid]; };
    auto I = [&](int p) -> int & { return li[(size_t)p * threads + tid]; };
    // (v, jv) orders after (m, jm): by distance, then index; a NaN orders after every number
    auto larger = [](T v, int jv, T m, int jm) {
      const bool vn = !(v == v), mn = !(m == m);
      if (vn != mn) return vn;
      if (vn) return jv > jm;
      return v > m || (v == m && jv > jm);
    };
    // sift (d, j) down from position `pos` of the max-heap [0, n)
    auto sift = [&](int pos, int n, T d, int j) {
      while (true) {
        int child = 2 * pos + 1;
        if (child >= n) break;
        T dc = D(child);
        int jc = I(child);
        if (child + 1 < n) {
          const T dr = D(child + 1);
          const int jr = I(child + 1);
          if (larger(dr, jr, dc, jc)) ++child, dc = dr, jc = jr;
        }
        if (!larger(dc, jc, d, j)) break;
        D(pos) = dc;
        I(pos) = jc;
        pos = child;
      }
      D(pos) = d;
      I(pos) = j;
    };
    auto heapify = [&](int n) {
      for (int p = n / 2 - 1; p >= 0; --p) sift(p, n, D(p), I(p));
    };

    for (int j0 = j_begin; j0 < j_end; j0 += KS_STAGE) {
      const int n = min(KS_STAGE, j_end - j0);
      __syncwarp();
      if (kl.cs == 1) {  // [N,3]: the stage is one contiguous run
        for (int e = lane; e < n * 3; e += 32) mystage[e] = rb[(int64_t)j0 * 3 + e];
      } else {           // [3,N]: three runs, interleaved into the stage
        for (int e = lane; e < n * 3; e += 32) {
          const int c = e / n, u = e - c * n;
          mystage[u * 3 + c] = rb[(int64_t)c * kl.cs + j0 + u];
        }
      }
      __syncwarp();
      if (valid) {
        for (int u = 0; u < n; ++u) {
          const T d = sqdist<T>(mystage[u * 3 + 0], mystage[u * 3 + 1], mystage[u * 3 + 2], qx, qy, qz);
          if (cnt < k) {  // the first k keys of the segment enter unconditionally
            D(cnt) = d;
            I(cnt) = j0 + u;
            if (++cnt == k) {
              heapify(k);
              heaped = true;
              worst = D(0);
            }
          } else if (d < worst || (worst != worst && d == d)) {
            // keys come in ascending index order: an equal distance never enters; a NaN at the root
            // (it orders after every number) gives way to any real distance
            sift(0, k, d, j0 + u);
            worst = D(0);
          }
        }
      }
    }
    if (valid) {  // heap -> ascending list (heap sort in place)
      if (!heaped) heapify(cnt);
      for (int n = cnt - 1; n > 0; --n) {
        const T dl = D(n);
        const int jl = I(n);
        D(n) = D(0);
        I(n) = I(0);
        sift(0, n, dl, jl);
      }
    }
    lcnt[tid] = cnt;
    __syncthreads();

    if (seg == 0 && valid) {
      T *od = dist + (b * N1 + i) * (int64_t)k;
      const int64_t orow = (b * N1 + i) * (int64_t)k;
      int pos[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) pos[s] = 0;
      for (int out = 0; out < k; ++out) {
        int bs = -1;
        T bd = 0;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          if (s < S && pos[s] < lcnt[s * 32 + lane]) {
            const T d = ld[(size_t)pos[s] * threads + s * 32 + lane];
            // strict "<": among equal distances the lower segment (lower indices) goes first; a NaN
            // head is only taken when nothing else is left
            if (bs < 0 || d < bd || (bd != bd && d == d)) {
              bs = s;
              bd = d;
            }
          }
        }
        if (bs < 0) break;  // cannot happen: the segments hold at least k keys together
        int bi = 0;
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (s == bs) {
            bi = li[(size_t)pos[s] * threads + s * 32 + lane];
            ++pos[s];
          }
        od[out] = bd;
        index.put(orow + out, bi);
      }
    }
    __syncthreads();
  }
}

}  // namespace

// Shared memory the split kernel needs for S warps per block.
static size_t knn_split_smem(int64_t k, int S, size_t elem) {
  const size_t threads = 32 * (size_t)S;
  return (size_t)k * threads * (elem + sizeof(int)) + (size_t)S * KS_STAGE * 3 * elem + threads * sizeof(int);
}

// Returns true and launches when the split kernel suits the problem; false = caller's own path.
bool knn_split_f64(const double *query, const double *key, int64_t B, int64_t N1, int64_t N2, int64_t k, double *dist,
                   IndexOut index, XyzLayout ql, XyzLayout kl, cudaStream_t st, int *rc) {
  const int64_t sms = sm_count();
  const int64_t warps = B * ((N1 + 31) / 32);
  if (k > 64 || warps >= sms * 32) return false;  // enough queries to fill the GPU one thread each
  int S = 8;
  while (S > 1 && (N2 / S < 4 * k || N2 / S < 128 || warps * (S / 2) >= sms * 32)) S /= 2;
  while (S >= 2 && knn_split_smem(k, S, sizeof(double)) > 200 * 1024) S /= 2;
  if (S < 2) return false;
  const size_t smem = knn_split_smem(k, S, sizeof(double));
  if (raise_smem_limit((const void *)knn_split_kernel<double>, (int)smem) !=
      cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  const int64_t cap = sms * 16;
  knn_split_kernel<double><<<(unsigned)(warps < cap ? warps : cap), 32 * S, smem, st>>>(
      query, key, B, (int)N1, (int)N2, (int)k, S, dist, index, warps, ql, kl);
  *rc = check_launch("knn_split_kernel");
  return true;
}

}  // namespace tk3d

TK3D_BOUNDS_TU(knn_split)
