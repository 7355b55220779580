// group_points: gather of per-point feature rows by neighbour index (forward) and the matching
// scatter-add (backward).  Both are memory-bound: the output (forward) or grad_output (backward)
// of B*C*N2*K elements dominates the traffic.
//
// Layout: in [B,C,N1], index [B,N2,K] -> out [B,C,N2,K].  With E = N2*K the output of one (b,c) is
// a contiguous run of E elements indexed by the SAME E indices for every channel, so a thread
// loads its indices once (the reference re-reads the int64 index tensor for every channel) and
// then walks the channels.
#include "rows.cuh"

namespace tk3d {

namespace {

constexpr int GP_THREADS = 256;
constexpr int GP_VEC = 4;                        // consecutive entries per thread
constexpr int GP_TILE = GP_THREADS * GP_VEC;     // entries per block

// Forward, direct gathers.  grid = (tiles of E, channel groups, B).
template <typename T>
__global__ void __launch_bounds__(GP_THREADS)
group_fwd_direct_kernel(const T *__restrict__ in, const int64_t *__restrict__ index, int64_t C, int64_t N1,
                        int64_t E, int64_t c_per_block, T *__restrict__ out, int32_t *__restrict__ status, int vec) {
  const int64_t b = blockIdx.z;
  const int64_t e0 = ((int64_t)blockIdx.x * GP_THREADS + threadIdx.x) * GP_VEC;
  if (e0 >= E) return;
  const int64_t c0 = (int64_t)blockIdx.y * c_per_block;
  const int64_t c1 = (c0 + c_per_block < C) ? c0 + c_per_block : C;
  const int64_t *ip = index + b * E + e0;
  const int n = (int)((E - e0) < GP_VEC ? (E - e0) : GP_VEC);
  int64_t id[GP_VEC];
  bool bad = false;
#pragma unroll
  for (int v = 0; v < GP_VEC; ++v) {
    id[v] = v < n ? ip[v] : 0;
    if (id[v] < 0 || id[v] >= N1) {
      id[v] = -1;
      bad |= v < n;
    }
  }
  if (bad && status) atomicOr(status, 1);
  const bool vec_ok = vec && n == GP_VEC;  // host checked: fp32, E % 4 == 0, 16-byte aligned base
  const T *src = in + (b * C + c0) * N1;
  T *dst = out + (b * C + c0) * E + e0;
#pragma unroll 4
  for (int64_t c = c0; c < c1; ++c, src += N1, dst += E) {
    T val[GP_VEC];
#pragma unroll
    for (int v = 0; v < GP_VEC; ++v) val[v] = id[v] >= 0 ? __ldg(src + id[v]) : (T)0;
    if constexpr (sizeof(T) == 4) {
      if (vec_ok) {
        // streaming store: the output is never re-read by this kernel
        __stcs(reinterpret_cast<float4 *>(dst), make_float4(val[0], val[1], val[2], val[3]));
        continue;
      }
    }
    {
      for (int v = 0; v < n; ++v) dst[v] = val[v];
    }
  }
}

// Backward, scatter with atomics; equal neighbouring indices (ball-query padding repeats the first
// hit) are merged before the atomic.
template <typename T>
__global__ void __launch_bounds__(GP_THREADS)
group_bwd_kernel(const T *__restrict__ gout, const int64_t *__restrict__ index, int64_t C, int64_t N1, int64_t E,
                 int64_t c_per_block, T *__restrict__ gin, int32_t *__restrict__ status, int vec) {
  const int64_t b = blockIdx.z;
  const int64_t e0 = ((int64_t)blockIdx.x * GP_THREADS + threadIdx.x) * GP_VEC;
  if (e0 >= E) return;
  const int64_t c0 = (int64_t)blockIdx.y * c_per_block;
  const int64_t c1 = (c0 + c_per_block < C) ? c0 + c_per_block : C;
  const int64_t *ip = index + b * E + e0;
  const int n = (int)((E - e0) < GP_VEC ? (E - e0) : GP_VEC);
  int64_t id[GP_VEC];
  bool bad = false;
#pragma unroll
  for (int v = 0; v < GP_VEC; ++v) {
    id[v] = v < n ? ip[v] : -1;
    if (v < n && (id[v] < 0 || id[v] >= N1)) {
      id[v] = -1;
      bad = true;
    }
  }
  if (bad && status) atomicOr(status, 1);
  const bool vec_ok = vec && n == GP_VEC;  // host checked: fp32, E % 4 == 0, 16-byte aligned base
  const T *src = gout + (b * C + c0) * E + e0;
  T *dst = gin + (b * C + c0) * N1;
#pragma unroll 2
  for (int64_t c = c0; c < c1; ++c, src += E, dst += N1) {
    T val[GP_VEC];
    bool loaded = false;
    if constexpr (sizeof(T) == 4) {
      if (vec_ok) {
        const float4 g = __ldcs(reinterpret_cast<const float4 *>(src));
        val[0] = g.x;
        val[1] = g.y;
        val[2] = g.z;
        val[3] = g.w;
        loaded = true;
      }
    }
    if (!loaded) {
#pragma unroll
      for (int v = 0; v < GP_VEC; ++v) val[v] = v < n ? src[v] : (T)0;
    }
    // Merge runs of equal indices, then one atomic per run.
    T acc = val[0];
    int64_t cur = id[0];
#pragma unroll
    for (int v = 1; v < GP_VEC; ++v) {
      if (id[v] == cur) {
        acc += val[v];
      } else {
        if (cur >= 0) atomicAdd(dst + cur, acc);
        cur = id[v];
        acc = val[v];
      }
    }
    if (cur >= 0) atomicAdd(dst + cur, acc);
  }
}

// How many channels one block walks: enough blocks to fill the GPU a few times over, but as few
// channel groups as possible so the indices are read once per group.
int64_t channels_per_block(int64_t tiles, int64_t B, int64_t C) {
  const int64_t want = (int64_t)sm_count() * 8;
  int64_t groups = (want + tiles * B - 1) / (tiles * B);
  if (groups < 1) groups = 1;
  if (groups > C) groups = C;
  return (C + groups - 1) / groups;
}

template <typename T>
int group_fwd_t(const T *in, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t E, T *out,
                int32_t *status, cudaStream_t st) {
  const int64_t tiles = (E + GP_TILE - 1) / GP_TILE;
  const int64_t cpb = channels_per_block(tiles, B, C);
  const int64_t groups = (C + cpb - 1) / cpb;
  TK3D_REQUIRE(tiles < (1LL << 31) && groups <= 65535 && B <= 65535, TK3D_ERR_SHAPE,
               "group_points: grid too large (B=%lld)", (long long)B);
  dim3 grid((unsigned)tiles, (unsigned)groups, (unsigned)B);
  const int vec = sizeof(T) == 4 && E % GP_VEC == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  group_fwd_direct_kernel<T><<<grid, GP_THREADS, 0, st>>>(in, index, C, N1, E, cpb, out, status, vec);
  return check_launch("group_fwd_direct_kernel");
}

template <typename T>
int group_bwd_t(const T *gout, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t E, T *gin,
                int32_t *status, cudaStream_t st) {
  TK3D_CUDA(cudaMemsetAsync(gin, 0, sizeof(T) * (size_t)(B * C * N1), st));
  if (E == 0) return TK3D_OK;
  const int64_t tiles = (E + GP_TILE - 1) / GP_TILE;
  const int64_t cpb = channels_per_block(tiles, B, C);
  const int64_t groups = (C + cpb - 1) / cpb;
  TK3D_REQUIRE(tiles < (1LL << 31) && groups <= 65535 && B <= 65535, TK3D_ERR_SHAPE,
               "group_points: grid too large (B=%lld)", (long long)B);
  dim3 grid((unsigned)tiles, (unsigned)groups, (unsigned)B);
  const int vec = sizeof(T) == 4 && E % GP_VEC == 0 && (reinterpret_cast<uintptr_t>(gout) & 15) == 0;
  group_bwd_kernel<T><<<grid, GP_THREADS, 0, st>>>(gout, index, C, N1, E, cpb, gin, status, vec);
  return check_launch("group_bwd_kernel");
}

int check_group_args(const char *what, const void *a, const int64_t *index, const void *o, int64_t B, int64_t C,
                     int64_t N1, int64_t N2, int64_t K, int dtype) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "%s: dtype %d", what, dtype);
  TK3D_REQUIRE(B >= 0 && C >= 0 && N1 >= 0 && N2 >= 0 && K >= 0, TK3D_ERR_SHAPE, "%s: negative size", what);
  TK3D_REQUIRE(N1 < (1LL << 31), TK3D_ERR_SHAPE, "%s: N1 limited to 2^31-1", what);
  (void)a;
  (void)index;
  (void)o;
  return TK3D_OK;
}

}  // namespace
}  // namespace tk3d

using namespace tk3d;

extern "C" size_t tk3d_group_fwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K, int dtype) {
  if (dtype != TK3D_F32 || B <= 0 || C <= 0 || N1 <= 0 || N2 <= 0 || K <= 0 || B > 65535) return 0;
  return rows_profitable(C, N1, N2 * K, 1) ? rows_scratch_bytes(B, C, N1) : 0;
}

extern "C" int tk3d_group_fwd(const void *in, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t N2,
                              int64_t K, void *out, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                              void *stream) {
  int rc = check_group_args("group_fwd", in, index, out, B, C, N1, N2, K, dtype);
  if (rc) return rc;
  const int64_t E = N2 * K;
  if (B * C * E == 0) return TK3D_OK;
  TK3D_REQUIRE(index && out && (in || N1 == 0), TK3D_ERR_NULL, "group_fwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F32) {
    const size_t want = tk3d_group_fwd_scratch_bytes(B, C, N1, N2, K, dtype);
    if (want != 0 && scratch != nullptr && scratch_bytes >= want)
      return gather_rows<1>((const float *)in, index, nullptr, B, C, N1, E, (float *)out, status, (float *)scratch, st);
    return group_fwd_t<float>((const float *)in, index, B, C, N1, E, (float *)out, status, st);
  }
  return group_fwd_t<double>((const double *)in, index, B, C, N1, E, (double *)out, status, st);
}

extern "C" size_t tk3d_group_bwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K, int dtype) {
  if (dtype != TK3D_F32 || C % 4 != 0 || (N2 * K) % 4 != 0 || (N1 + 31) / 32 > 65535) return 0;
  return tk3d_group_fwd_scratch_bytes(B, C, N1, N2, K, dtype);
}

extern "C" int tk3d_group_bwd(const void *gout, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t N2,
                              int64_t K, void *gin, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                              void *stream) {
  int rc = check_group_args("group_bwd", gout, index, gin, B, C, N1, N2, K, dtype);
  if (rc) return rc;
  const int64_t E = N2 * K;
  if (B * C * N1 == 0) return TK3D_OK;
  TK3D_REQUIRE(gin && (E == 0 || (index && gout)), TK3D_ERR_NULL, "group_bwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F32) {
    const size_t want = tk3d_group_bwd_scratch_bytes(B, C, N1, N2, K, dtype);
    if (want != 0 && scratch != nullptr && scratch_bytes >= want && rows_vec_ok(C, E, gout, scratch))
      return scatter_rows<1>((const float *)gout, index, nullptr, B, C, N1, E, (float *)gin, status, (float *)scratch,
                             st);
    return group_bwd_t<float>((const float *)gout, index, B, C, N1, E, (float *)gin, status, st);
  }
  return group_bwd_t<double>((const double *)gout, index, B, C, N1, E, (double *)gin, status, st);
}
