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
template <typename T, typename IndexT>
__global__ void __launch_bounds__(GP_THREADS)
group_fwd_direct_kernel(const T *__restrict__ in, const IndexT *__restrict__ index, int64_t C, int64_t N1,
                        int64_t E, int64_t c_per_block, T *__restrict__ out, int32_t *__restrict__ status, int vec) {
  const int64_t b = blockIdx.z;
  const int64_t e0 = ((int64_t)blockIdx.x * GP_THREADS + threadIdx.x) * GP_VEC;
  if (e0 >= E) return;
  const int64_t c0 = (int64_t)blockIdx.y * c_per_block;
  const int64_t c1 = (c0 + c_per_block < C) ? c0 + c_per_block : C;
  const IndexT *ip = index + b * E + e0;
  const int n = (int)((E - e0) < GP_VEC ? (E - e0) : GP_VEC);
  int64_t id[GP_VEC];
  bool bad = false;
#pragma unroll
  for (int v = 0; v < GP_VEC; ++v) {
    id[v] = v < n ? (int64_t)ip[v] : 0;
    if (id[v] < 0 || id[v] >= N1) {
      id[v] = -1;
      bad |= v < n;
    }
  }
  if (bad && status) atomicOr(status, 1);
  const bool vec_ok = vec && n == GP_VEC;  // host checked: E % 4 == 0, 16-byte aligned base
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
    } else {
      if (vec_ok) {  // float64: two 16-byte stores instead of four scalar ones
        __stcs(reinterpret_cast<double2 *>(dst), make_double2(val[0], val[1]));
        __stcs(reinterpret_cast<double2 *>(dst) + 1, make_double2(val[2], val[3]));
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

// ---------------------------------------------------------------------------------------------
// Channel-row forward kernel (clouds whose N1 features fit shared memory twice): no transposed
// copy of the features, no scratch.  (The mirror image for the backward -- gradient rows
// accumulated with shared-memory reductions -- was measured slower than the vector reductions
// into a transposed accumulator, 0.18 against 0.12 ms on 32 x 64 x 8192 <- 32768 entries: a
// shared-memory float reduction per element is the bottleneck.)
//
// A block owns a chunk of the E = N2*K index entries of one cloud -- each thread keeps
// its entries' indices in registers for the whole block -- and walks a group of channels.  The
// N1 features of a channel are one contiguous row of the [B,C,N1] tensor: the row is brought into
// shared memory with 16-byte cp.async copies, double buffered so that the next row lands while
// the current one is gathered, and the gather itself is a shared-memory read per output element
// followed by 16-byte streaming stores of four consecutive entries.  HBM sees every feature and
// every index once (the row re-reads of neighbouring blocks hit L2) and the output once.
// An index outside [0,N1) reads the zero kept behind the row.
constexpr int CR_THREADS = 256;

__device__ __forceinline__ void cr_cp_async16(void *smem, const void *gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cr_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void cr_cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

// R rounds of four consecutive entries per thread: a block covers CR_THREADS * 4 * R entries.
template <typename T, typename IndexT, int R, bool VEC>
__global__ void __launch_bounds__(CR_THREADS)
group_fwd_chanrow_kernel(const T *__restrict__ in, const IndexT *__restrict__ index, int C, int N1, int64_t E,
                         int cg, T *__restrict__ out, int32_t *__restrict__ status) {
  extern __shared__ __align__(16) unsigned char cr_raw[];
  T *cr_rows = reinterpret_cast<T *>(cr_raw);  // [2][N1 + 4]; slots N1..N1+3 of each hold 0
  constexpr int PER16 = 16 / (int)sizeof(T);   // elements per 16-byte copy
  const int tid = threadIdx.x;
  const int64_t b = blockIdx.z;
  const int c0 = blockIdx.y * cg, c1 = min(C, c0 + cg);
  const int64_t e0 = (int64_t)blockIdx.x * (CR_THREADS * 4 * R);
  const int stride = N1 + 4;

  int id[R][4];
  bool bad = false;
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int64_t e = e0 + (int64_t)(r * CR_THREADS + tid) * 4 + v;
      int64_t j = e < E ? (int64_t)index[b * E + e] : 0;
      if (j < 0 || j >= N1) {
        j = N1;  // the zero behind the row
        bad = true;
      }
      id[r][v] = (int)j;
    }
  }
  if (bad && status) atomicOr(status, 1);
  if (tid < 8) cr_rows[(tid >> 2) * stride + N1 + (tid & 3)] = (T)0;

  const T *src = in + (b * C + c0) * (int64_t)N1;
  auto stage = [&](int c, int buf) {
    const T *g = src + (int64_t)(c - c0) * N1;
    T *d = cr_rows + buf * stride;
    for (int q = tid; q < N1 / PER16; q += CR_THREADS) cr_cp_async16(d + PER16 * q, g + PER16 * q);
    cr_cp_commit();
  };
  stage(c0, 0);
  for (int c = c0; c < c1; ++c) {
    const int buf = (c - c0) & 1;
    if (c + 1 < c1) {
      stage(c + 1, buf ^ 1);  // the other buffer was released by the barrier that ended the last round
      cr_cp_wait<1>();
    } else {
      cr_cp_wait<0>();
    }
    __syncthreads();
    const T *row = cr_rows + buf * stride;
    T *o = out + (b * C + c) * E;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t e = e0 + (int64_t)(r * CR_THREADS + tid) * 4;
      if (e >= E) break;
      const T v0 = row[id[r][0]], v1 = row[id[r][1]], v2 = row[id[r][2]], v3 = row[id[r][3]];
      if (VEC) {
        if constexpr (sizeof(T) == 4) {
          __stcs(reinterpret_cast<float4 *>(o + e), make_float4(v0, v1, v2, v3));
        } else {
          __stcs(reinterpret_cast<double2 *>(o + e), make_double2(v0, v1));
          __stcs(reinterpret_cast<double2 *>(o + e) + 1, make_double2(v2, v3));
        }
      } else {
        o[e] = v0;
        if (e + 1 < E) o[e + 1] = v1;
        if (e + 2 < E) o[e + 2] = v2;
        if (e + 3 < E) o[e + 3] = v3;
      }
    }
    __syncthreads();
  }
}

// Largest cloud the channel-row kernels take: two rows (forward) must fit the 227 KB of an SM
// (24576 floats or 12288 doubles).
constexpr int64_t CR_MAX_ROW_BYTES = 24576 * 4;

inline bool chanrow_ok(const void *in, int64_t B, int64_t C, int64_t N1, int64_t E, int64_t elem = 4) {
  return N1 >= 256 && N1 % 4 == 0 && N1 * elem <= CR_MAX_ROW_BYTES && E >= 1024 && B <= 65535 && C <= 65535 &&
         (reinterpret_cast<uintptr_t>(in) & 15) == 0;
}

template <typename T, typename IndexT>
int group_fwd_chanrow(const T *in, const IndexT *index, int64_t B, int64_t C, int64_t N1, int64_t E, T *out,
                      int32_t *status, cudaStream_t st) {
  // entries per block: 8192 when that still leaves enough blocks, else 4096
  const int64_t sms = sm_count();
  const bool big = B * ((E + 8191) / 8192) * 4 >= 3 * sms;
  const int64_t ech = big ? 8192 : 4096;
  const int64_t chunks = (E + ech - 1) / ech;
  // channel groups: enough blocks for about three per SM, as few groups as possible beyond that
  int64_t groups = (3 * sms + B * chunks - 1) / (B * chunks);
  groups = groups < 1 ? 1 : (groups > C ? C : groups);
  const int cg = (int)((C + groups - 1) / groups);
  groups = (C + cg - 1) / cg;
  TK3D_REQUIRE(chunks < (1LL << 31), TK3D_ERR_SHAPE, "group_points: too many entries");
  const size_t smem = (size_t)2 * (N1 + 4) * sizeof(T);
  dim3 grid((unsigned)chunks, (unsigned)groups, (unsigned)B);
  const bool vec = E % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
#define TK3D_CR_LAUNCH(RR, VV)                                                                                   \
  {                                                                                                              \
    TK3D_CUDA(raise_smem_limit((const void *)group_fwd_chanrow_kernel<T, IndexT, RR, VV>, (int)smem));             \
    group_fwd_chanrow_kernel<T, IndexT, RR, VV><<<grid, CR_THREADS, smem, st>>>(in, index, (int)C, (int)N1, E, cg, \
                                                                                out, status);                       \
  }
  if (big) {
    if (vec) TK3D_CR_LAUNCH(8, true) else TK3D_CR_LAUNCH(8, false)
  } else {
    if (vec) TK3D_CR_LAUNCH(4, true) else TK3D_CR_LAUNCH(4, false)
  }
#undef TK3D_CR_LAUNCH
  return check_launch("group_fwd_chanrow_kernel");
}

// How many channels one block walks: enough blocks to fill the GPU a few times over, but as few
// channel groups as possible so the indices are read once per group.
int64_t channels_per_block(int64_t tiles, int64_t B, int64_t C, int mult = 8) {
  const int64_t want = (int64_t)sm_count() * mult;
  int64_t groups = (want + tiles * B - 1) / (tiles * B);
  if (groups < 1) groups = 1;
  if (groups > C) groups = C;
  return (C + groups - 1) / groups;
}

template <typename T, typename IndexT>
int group_fwd_t(const T *in, const IndexT *index, int64_t B, int64_t C, int64_t N1, int64_t E, T *out,
                int32_t *status, cudaStream_t st) {
  const int64_t tiles = (E + GP_TILE - 1) / GP_TILE;
  const int64_t cpb = channels_per_block(tiles, B, C);
  const int64_t groups = (C + cpb - 1) / cpb;
  TK3D_REQUIRE(tiles < (1LL << 31) && groups <= 65535 && B <= 65535, TK3D_ERR_SHAPE,
               "group_points: grid too large (B=%lld)", (long long)B);
  dim3 grid((unsigned)tiles, (unsigned)groups, (unsigned)B);
  const int vec = E % GP_VEC == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
  group_fwd_direct_kernel<T, IndexT><<<grid, GP_THREADS, 0, st>>>(in, index, C, N1, E, cpb, out, status, vec);
  return check_launch("group_fwd_direct_kernel");
}

template <typename T>
int group_bwd_t(const T *gout, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t E, T *gin,
                int32_t *status, cudaStream_t st) {
  TK3D_CUDA(cudaMemsetAsync(gin, 0, sizeof(T) * (size_t)(B * C * N1), st));
  if (E == 0) return TK3D_OK;
  const int64_t tiles = (E + GP_TILE - 1) / GP_TILE;
  // many small blocks suit the atomics (float64, 8 x 64 x 1024 <- 512 x 32: 0.059 -> 0.053 ms)
  const int64_t cpb = channels_per_block(tiles, B, C, 128);
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
  // shapes the channel-row kernels take need no scratch (given 16-byte aligned features; an
  // unaligned tensor then runs the direct kernel)
  if (chanrow_ok(nullptr, B, C, N1, N2 * K)) return 0;
  return rows_profitable(C, N1, N2 * K, 1) ? rows_scratch_bytes(B, C, N1) : 0;
}

template <typename IndexT>
static int group_fwd_impl(const void *in, const IndexT *index, int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K,
                          void *out, int32_t *status, void *scratch, size_t scratch_bytes, int dtype, void *stream) {
  int rc = check_group_args("group_fwd", in, nullptr, out, B, C, N1, N2, K, dtype);
  if (rc) return rc;
  const int64_t E = N2 * K;
  if (B * C * E == 0) return TK3D_OK;
  TK3D_REQUIRE(index && out && (in || N1 == 0), TK3D_ERR_NULL, "group_fwd: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == TK3D_F32) {
    if (chanrow_ok(in, B, C, N1, E))
      return group_fwd_chanrow<float, IndexT>((const float *)in, index, B, C, N1, E, (float *)out, status, st);
    const size_t want = tk3d_group_fwd_scratch_bytes(B, C, N1, N2, K, dtype);
    const size_t rows = rows_profitable(C, N1, E, 1) && B <= 65535 ? rows_scratch_bytes(B, C, N1) : 0;
    (void)want;
    if (rows != 0 && scratch != nullptr && scratch_bytes >= rows)
      return gather_rows<1, IndexT>((const float *)in, index, nullptr, B, C, N1, E, (float *)out, status,
                                    (float *)scratch, st);
    return group_fwd_t<float, IndexT>((const float *)in, index, B, C, N1, E, (float *)out, status, st);
  }
  if (chanrow_ok(in, B, C, N1, E, 8))
    return group_fwd_chanrow<double, IndexT>((const double *)in, index, B, C, N1, E, (double *)out, status, st);
  return group_fwd_t<double, IndexT>((const double *)in, index, B, C, N1, E, (double *)out, status, st);
}

extern "C" int tk3d_group_fwd(const void *in, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t N2,
                              int64_t K, void *out, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                              void *stream) {
  TK3D_RANGE("tk3d_group_fwd");
  return group_fwd_impl<int64_t>(in, index, B, C, N1, N2, K, out, status, scratch, scratch_bytes, dtype, stream);
}

extern "C" int tk3d_group_fwd_layout(const void *in, const void *index, int index_dtype, int64_t B, int64_t C,
                                     int64_t N1, int64_t N2, int64_t K, void *out, int32_t *status, void *scratch,
                                     size_t scratch_bytes, int dtype, void *stream) {
  TK3D_RANGE("tk3d_group_fwd_layout");
  TK3D_REQUIRE(index_dtype == TK3D_I64 || index_dtype == TK3D_I32, TK3D_ERR_DTYPE, "group_fwd: index_dtype %d",
               index_dtype);
  if (index_dtype == TK3D_I32)
    return group_fwd_impl<int32_t>(in, (const int32_t *)index, B, C, N1, N2, K, out, status, scratch, scratch_bytes,
                                   dtype, stream);
  return group_fwd_impl<int64_t>(in, (const int64_t *)index, B, C, N1, N2, K, out, status, scratch, scratch_bytes,
                                 dtype, stream);
}

extern "C" int tk3d_group_fwd_rows(const void *rows, const void *index, int index_dtype, int64_t B, int64_t C,
                                   int64_t N1, int64_t N2, int64_t K, void *out, int32_t *status, int dtype,
                                   void *stream) {
  TK3D_RANGE("tk3d_group_fwd_rows");
  int rc = check_group_args("group_fwd_rows", rows, nullptr, out, B, C, N1, N2, K, dtype);
  if (rc) return rc;
  TK3D_REQUIRE(dtype == TK3D_F32, TK3D_ERR_DTYPE, "group_fwd_rows: float32 only (dtype %d)", dtype);
  TK3D_REQUIRE(index_dtype == TK3D_I64 || index_dtype == TK3D_I32, TK3D_ERR_DTYPE, "group_fwd_rows: index_dtype %d",
               index_dtype);
  TK3D_REQUIRE(C <= ROWS_MAX_C && B <= 65535, TK3D_ERR_SHAPE, "group_fwd_rows: C <= %d and B <= 65535 required",
               ROWS_MAX_C);
  const int64_t E = N2 * K;
  if (B * C * E == 0) return TK3D_OK;
  TK3D_REQUIRE(index && out && (rows || N1 == 0), TK3D_ERR_NULL, "group_fwd_rows: a pointer is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  if (index_dtype == TK3D_I32)
    return gather_from_rows<1, int32_t>((const float *)rows, (const int32_t *)index, nullptr, B, C, N1, E,
                                        (float *)out, status, st);
  return gather_from_rows<1, int64_t>((const float *)rows, (const int64_t *)index, nullptr, B, C, N1, E, (float *)out,
                                      status, st);
}

extern "C" size_t tk3d_group_bwd_scratch_bytes(int64_t B, int64_t C, int64_t N1, int64_t N2, int64_t K, int dtype) {
  if (dtype != TK3D_F32 || B <= 0 || C <= 0 || N1 <= 0 || N2 <= 0 || K <= 0 || B > 65535) return 0;
  if (C % 4 != 0 || (N2 * K) % 4 != 0 || (N1 + 31) / 32 > 65535) return 0;
  return rows_profitable(C, N1, N2 * K, 1) ? rows_scratch_bytes(B, C, N1) : 0;
}

extern "C" int tk3d_group_bwd(const void *gout, const int64_t *index, int64_t B, int64_t C, int64_t N1, int64_t N2,
                              int64_t K, void *gin, int32_t *status, void *scratch, size_t scratch_bytes, int dtype,
                              void *stream) {
  TK3D_RANGE("tk3d_group_bwd");
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

TK3D_BOUNDS_TU(group)
