// Farthest point sampling.
//
// The algorithm is a chain of S-1 dependent steps per cloud (update every point's distance to the
// selected set, pick the arg-max), so the design goal is latency per step, not bandwidth:
//
//  * fp32, N <= 16384 ("resident" kernel): one persistent CTA per cloud keeps every point and its
//    running minimum distance in REGISTERS for the whole call (up to 8 points per thread), plus a
//    copy of the coordinates in shared memory from which the newly selected point is broadcast.
//    Clouds of 8193 to 16384 points keep 16 running minima per thread in registers and read the
//    coordinates from the shared-memory copy (192 KB at most) in every step.
//    A step is: P exact distance updates per thread, a block-wide maximum of the running minima
//    (REDUX, one shared-memory exchange, REDUX), and the lowest index holding that maximum.
//    Clouds of up to 4096 points, and large batches of clouds up to 16384 points (more than about
//    half a cloud per SM).
//  * fp64, N <= 8192: the same persistent structure with the coordinates in shared memory and up to
//    8 running minima per thread; the block maximum is taken on the 64-bit pattern in two REDUX steps.
//    (Few clouds of 2049 to 8192 points and every cloud of 8193 to 131072 points: clusters, fps_cluster.cu.)
//  * fp32, 16385 to 262144 points (and few clouds of 4097 to 16384): a thread-block cluster per cloud,
//    fps_cluster.cu.
//  * any other case ("streaming" kernel): points are re-read from global memory (L1/L2 resident)
//    and the running minimum lives in a caller-provided global scratch array.
//
// Arg-max rule: highest running minimum distance, lowest index among exact ties.  Distances are
// non-negative, so their IEEE bit patterns order like unsigned integers and the pair
// (distance bits, ~index) can be maximised with integer reductions.
#include "tk3d_common.cuh"

namespace tk3d {

namespace {

constexpr int FPS_MAX_THREADS = 1024;

// ---- resident kernel (fp32) ------------------------------------------------------------------
// A step inside the SM is bound by issue slots and the half-rate ALU pipe rather than by latency,
// so the per-point work on that pipe is kept to one min and one max: threads track only their
// largest running minimum, the block reduces the VALUE (REDUX + one shared-memory exchange), and
// only the threads that hold the winning value look up their lowest index with it and publish it
// with a shared-memory atomicMin.  That costs a second barrier per step but removes the
// compare-and-two-selects per point of an index-carrying arg-max (0.835 ms against 0.885 ms for
// 32 clouds of 8192 points).  Points are held two per float2 register pair.
// The distance runs on the packed FP32 instructions of sm_100 (two points per instruction): the
// step is bound by instruction issue, and eight packed operations per two points replace sixteen
// scalar ones (0.85 -> 0.70 ms for 32 clouds of 8192 points).  Bit-exactness needs care: a packed
// add fed by a packed multiply comes out contracted into one fused multiply-add -- with explicit
// .rn on both, as intrinsics or as inline PTX alike -- which changes the last bit of about one
// distance in five and flips exactly tied winners.  The sums are therefore written fma(x, one, y)
// with `one` = 1.0f passed as a kernel argument: round(x * 1 + y) = round(x + y), and an FMA with
// an unknown multiplier cannot be merged with the multiplies that produced x and y.
// REG = false (clouds of 8193 to 16384 points, 16 per thread): only the running minima stay in
// registers, the coordinates are read from the shared-memory copy in every step.
template <int P2, bool REG = true>
__global__ void __launch_bounds__(FPS_MAX_THREADS)
fps_resident_kernel(const float *__restrict__ points, int N, int S, int64_t *__restrict__ index, int ps, int cs,
                    float *__restrict__ sampled, float one) {
  extern __shared__ float sxyz[];  // [3*N] copy of the cloud
  __shared__ unsigned slots[2][32];
  __shared__ int s_idx[2];
  const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = T >> 5;
  const float *pts = points + (int64_t)blockIdx.x * N * 3;
  int64_t *out = index + (int64_t)blockIdx.x * S;

  // Point j, coordinate d sits at pts[j*ps + d*cs]: (3, 1) for [N,3] clouds, (1, N) for [3,N].
  if (cs == 1) {
    for (int e = tid; e < 3 * N; e += T) sxyz[e] = pts[e];
  } else {
    for (int e = tid; e < 3 * N; e += T) {
      const int d = e / N, j = e - d * N;
      sxyz[3 * j + d] = pts[e];
    }
  }
  if (tid < 2) s_idx[tid] = 0x7fffffff;
  __syncthreads();

  // Point (i, h) of this thread is j = (2*i + h) * T + tid: ascending in (i, h).
  float2 px[REG ? P2 : 1], py[REG ? P2 : 1], pz[REG ? P2 : 1], md[P2];
  const float qnan = __int_as_float(0x7fc00000), pinf = __int_as_float(0x7f800000);
#pragma unroll
  for (int i = 0; i < P2; ++i) {
    const int j0 = (2 * i) * T + tid, j1 = (2 * i + 1) * T + tid;
    if (REG) {
      px[i].x = j0 < N ? sxyz[3 * j0 + 0] : qnan;
      py[i].x = j0 < N ? sxyz[3 * j0 + 1] : qnan;
      pz[i].x = j0 < N ? sxyz[3 * j0 + 2] : qnan;
      px[i].y = j1 < N ? sxyz[3 * j1 + 0] : qnan;
      py[i].y = j1 < N ? sxyz[3 * j1 + 1] : qnan;
      pz[i].y = j1 < N ? sxyz[3 * j1 + 2] : qnan;
    }
    md[i].x = j0 < N ? pinf : 0.f;  // padding: distance 0, NaN coordinates keep it there
    md[i].y = j1 < N ? pinf : 0.f;
  }

  int cur = 0;
  if (tid == 0) out[0] = 0;
  const float2 one2 = make_float2(one, one);
  for (int it = 1; it < S; ++it) {
    const int par = it & 1;
    const float cx = sxyz[3 * cur + 0], cy = sxyz[3 * cur + 1], cz = sxyz[3 * cur + 2];
    const float2 ncx = make_float2(-cx, -cx), ncy = make_float2(-cy, -cy), ncz = make_float2(-cz, -cz);
    float bm = 0.f;
#pragma unroll
    for (int i = 0; i < P2; ++i) {
      float2 qx, qy, qz;
      if (REG) {
        qx = px[i], qy = py[i], qz = pz[i];
      } else {
        // beyond N the running minimum is 0 and stays 0 whatever is read (the index is clamped)
        const int j0 = min((2 * i) * T + tid, N - 1), j1 = min((2 * i + 1) * T + tid, N - 1);
        qx = make_float2(sxyz[3 * j0], sxyz[3 * j1]);
        qy = make_float2(sxyz[3 * j0 + 1], sxyz[3 * j1 + 1]);
        qz = make_float2(sxyz[3 * j0 + 2], sxyz[3 * j1 + 2]);
      }
      // p - c as p + (-c) (identical in IEEE arithmetic), squares by packed multiplies, the two
      // sums as fma(x, one, y): see the note above the kernel.
      const float2 dx = __fadd2_rn(qx, ncx), dy = __fadd2_rn(qy, ncy), dz = __fadd2_rn(qz, ncz);
      const float2 d = __ffma2_rn(__ffma2_rn(__fmul2_rn(dx, dx), one2, __fmul2_rn(dy, dy)), one2, __fmul2_rn(dz, dz));
      md[i].x = fminf(md[i].x, d.x);
      md[i].y = fminf(md[i].y, d.y);
      asm("max.f32 %0, %0, %1, %2;" : "+f"(bm) : "f"(md[i].x), "f"(md[i].y));  // three-input maximum
    }
    const unsigned bits = __float_as_uint(bm);
    unsigned gb = __reduce_max_sync(0xffffffffu, bits);
    if (nwarps > 1) {
      if (lane == 0) slots[par][warp] = gb;
      __syncthreads();
      gb = __reduce_max_sync(0xffffffffu, lane < nwarps ? slots[par][lane] : 0u);
    }
    // Re-arm the other slot for the next step: all its readers are past the barrier above.
    if (nwarps > 1 && tid == 0) s_idx[par ^ 1] = 0x7fffffff;
    // Threads that hold the winning value look up their lowest point with it and publish the
    // smallest such index.
    if (bits == gb) {
      int mine = 0x7fffffff;
#pragma unroll
      for (int i = P2 - 1; i >= 0; --i) {
        if (md[i].y == bm) mine = (2 * i + 1) * T + tid;
        if (md[i].x == bm) mine = (2 * i) * T + tid;
      }
      atomicMin(&s_idx[par], mine);
    }
    __syncthreads();
    cur = s_idx[par];
    if (nwarps == 1) {
      __syncwarp();
      if (tid == 0) s_idx[par ^ 1] = 0x7fffffff;
    }
    if (tid == 0) out[it] = cur;
  }
  // Optional epilogue: coordinates of the samples, in the layout of the input ([S,3] or [3,S]).
  if (sampled != nullptr) {
    __syncthreads();  // makes thread 0's index stores visible to the block
    float *sm = sampled + (int64_t)blockIdx.x * S * 3;
    const int sps = cs == 1 ? 3 : 1, scs = cs == 1 ? 1 : S;
    for (int e = tid; e < 3 * S; e += T) {
      const int s = e / 3, d = e - 3 * s;
      sm[s * sps + d * scs] = sxyz[3 * (int)out[s] + d];
    }
  }
}

// ---- resident kernel, fp64 ------------------------------------------------------------------------
// Same structure for double precision clouds of up to 8192 points: coordinates in shared memory
// (24 bytes per point), up to 8 running minima per thread in registers.  Distances are
// non-negative, so their bit patterns order like unsigned 64-bit integers; a warp takes the maximum
// of the high words, then of the low words among the lanes that hold that high word.
constexpr int64_t FPS_RESIDENT64_MAX_N = 8192;

__device__ __forceinline__ unsigned long long fps_warp_max64(unsigned long long v) {
  const unsigned hi = (unsigned)(v >> 32), lo = (unsigned)v;
  const unsigned whi = __reduce_max_sync(0xffffffffu, hi);
  const unsigned wlo = __reduce_max_sync(0xffffffffu, hi == whi ? lo : 0u);
  return ((unsigned long long)whi << 32) | wlo;
}

template <int P>
__global__ void __launch_bounds__(FPS_MAX_THREADS)
fps_resident64_kernel(const double *__restrict__ points, int N, int S, int64_t *__restrict__ index, int ps, int cs,
                      double *__restrict__ sampled) {
  extern __shared__ double dxyz[];  // [3*N] copy of the cloud
  __shared__ unsigned long long slots64[2][32];
  __shared__ int s_idx[2];
  const int tid = threadIdx.x, T = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = T >> 5;
  const double *pts = points + (int64_t)blockIdx.x * N * 3;
  int64_t *out = index + (int64_t)blockIdx.x * S;
  if (cs == 1) {
    for (int e = tid; e < 3 * N; e += T) dxyz[e] = pts[e];
  } else {
    for (int e = tid; e < 3 * N; e += T) {
      const int d = e / N, j = e - d * N;
      dxyz[3 * j + d] = pts[e];
    }
  }
  if (tid < 2) s_idx[tid] = 0x7fffffff;
  __syncthreads();

  // Point i of this thread is j = i * T + tid; beyond N the running minimum is 0 and stays 0.
  double md[P];
#pragma unroll
  for (int i = 0; i < P; ++i) md[i] = (i * T + tid) < N ? Exact<double>::inf() : 0.0;

  int cur = 0;
  if (tid == 0) out[0] = 0;
  for (int it = 1; it < S; ++it) {
    const int par = it & 1;
    const double cx = dxyz[3 * cur + 0], cy = dxyz[3 * cur + 1], cz = dxyz[3 * cur + 2];
    double bm = 0.0;
#pragma unroll
    for (int i = 0; i < P; ++i) {
      const int j = min(i * T + tid, N - 1);
      const double d = sqdist<double>(dxyz[3 * j], dxyz[3 * j + 1], dxyz[3 * j + 2], cx, cy, cz);
      md[i] = fmin(md[i], d);
      bm = fmax(bm, md[i]);
    }
    const unsigned long long bits = (unsigned long long)__double_as_longlong(bm);
    unsigned long long gb = fps_warp_max64(bits);
    if (nwarps > 1) {
      if (lane == 0) slots64[par][warp] = gb;
      __syncthreads();
      gb = fps_warp_max64(lane < nwarps ? slots64[par][lane] : 0ull);
    }
    if (nwarps > 1 && tid == 0) s_idx[par ^ 1] = 0x7fffffff;
    if (bits == gb) {
      int mine = 0x7fffffff;
#pragma unroll
      for (int i = P - 1; i >= 0; --i)
        if (md[i] == bm) mine = i * T + tid;
      atomicMin(&s_idx[par], mine);
    }
    __syncthreads();
    cur = s_idx[par];
    if (nwarps == 1) {
      __syncwarp();
      if (tid == 0) s_idx[par ^ 1] = 0x7fffffff;
    }
    if (tid == 0) out[it] = cur;
  }
  if (sampled != nullptr) {
    __syncthreads();
    double *sm = sampled + (int64_t)blockIdx.x * S * 3;
    const int sps = cs == 1 ? 3 : 1, scs = cs == 1 ? 1 : S;
    for (int e = tid; e < 3 * S; e += T) {
      const int s = e / 3, d = e - 3 * s;
      sm[s * sps + d * scs] = dxyz[3 * (int)out[s] + d];
    }
  }
}

// ---- streaming kernel (any type, any N) ------------------------------------------------------
template <typename T>
__device__ __forceinline__ unsigned long long dist_key(T v);
template <>
__device__ __forceinline__ unsigned long long dist_key<float>(float v) {
  return (unsigned long long)__float_as_uint(v) << 32;
}
template <>
__device__ __forceinline__ unsigned long long dist_key<double>(double v) {
  return (unsigned long long)__double_as_longlong(v);
}

template <typename T>
__global__ void __launch_bounds__(FPS_MAX_THREADS)
fps_streaming_kernel(const T *__restrict__ points, int64_t N, int64_t S, int64_t *__restrict__ index,
                     T *__restrict__ min_dist, int64_t ps = 3, int64_t cs = 1, T *__restrict__ sampled = nullptr) {
  // Arg-max over (distance key, ~index) with 64-bit keys for the distance and a separate 64-bit
  // word for the index, reduced through shared memory.
  __shared__ unsigned long long skey[2][32];
  __shared__ unsigned long long sidx[2][32];
  const int tid = threadIdx.x, Tn = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = Tn >> 5;
  const T *pts = points + (int64_t)blockIdx.x * N * 3;
  T *md = min_dist + (int64_t)blockIdx.x * N;
  int64_t *out = index + (int64_t)blockIdx.x * S;

  int64_t cur = 0;
  if (tid == 0) out[0] = 0;
  for (int64_t it = 1; it < S; ++it) {
    const T cx = pts[ps * cur], cy = pts[ps * cur + cs], cz = pts[ps * cur + 2 * cs];
    unsigned long long bk = 0;
    unsigned long long bi = ~0ull;  // holds ~index so that max() prefers the lowest index
    bool any = false;
    for (int64_t j = tid; j < N; j += Tn) {
      const T d = sqdist<T>(pts[ps * j], pts[ps * j + cs], pts[ps * j + 2 * cs], cx, cy, cz);
      T m = (it == 1) ? Exact<T>::inf() : md[j];
      if (d < m) m = d;
      md[j] = m;
      const unsigned long long k = dist_key<T>(m);
      if (!any || k > bk) {
        bk = k;
        bi = ~(unsigned long long)j;
        any = true;
      }
    }
    if (!any) {
      bk = 0;
      bi = 0;  // loses every tie against a real point
    }
    // warp reduce (lexicographic max on (bk, bi))
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long ok = __shfl_xor_sync(0xffffffffu, bk, o);
      const unsigned long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ok > bk || (ok == bk && oi > bi)) {
        bk = ok;
        bi = oi;
      }
    }
    if (lane == 0) {
      skey[it & 1][warp] = bk;
      sidx[it & 1][warp] = bi;
    }
    __syncthreads();
    bk = lane < nwarps ? skey[it & 1][lane] : 0ull;
    bi = lane < nwarps ? sidx[it & 1][lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long ok = __shfl_xor_sync(0xffffffffu, bk, o);
      const unsigned long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ok > bk || (ok == bk && oi > bi)) {
        bk = ok;
        bi = oi;
      }
    }
    cur = (int64_t)(~bi);
    if (tid == 0) out[it] = cur;
  }
  if (sampled != nullptr) {
    __syncthreads();  // makes thread 0's index stores visible to the block
    T *sm = sampled + (int64_t)blockIdx.x * S * 3;
    const int64_t sps = cs == 1 ? 3 : 1, scs = cs == 1 ? 1 : S;
    for (int64_t e = tid; e < 3 * S; e += Tn) {
      const int64_t s = e / 3, d = e - 3 * s;
      sm[s * sps + d * scs] = pts[ps * out[s] + d * cs];
    }
  }
}

constexpr int64_t FPS_RESIDENT_MAX_N = 16384;  // 3*N floats of shared memory: 192 KB

int threads_for(int64_t N) {
  int t = 32;
  while (t < FPS_MAX_THREADS && t < N) t <<= 1;
  return t;
}

}  // namespace

}  // namespace tk3d

namespace tk3d {
bool fps_cluster_f32(const float *points, int64_t B, int64_t N, int64_t S, int ps, int64_t cs, int64_t *index,
                     float *sampled, cudaStream_t st, int *rc);
bool fps_cluster_f64(const double *points, int64_t B, int64_t N, int64_t S, int ps, int64_t cs, int64_t *index,
                     double *sampled, cudaStream_t st, int *rc);
}

using namespace tk3d;

extern "C" size_t tk3d_fps_scratch_bytes(int64_t B, int64_t N, int dtype) {
  if (B <= 0 || N <= 0) return 0;
  if (dtype == TK3D_F32 && N <= FPS_RESIDENT_MAX_N) return 0;
  if (dtype == TK3D_F64 && N <= FPS_RESIDENT64_MAX_N) return 0;
  return (size_t)B * (size_t)N * (dtype == TK3D_F64 ? 8 : 4);
}

static int fps_impl(const void *points, int64_t B, int64_t N, int64_t S, int channel_first, int64_t *index,
                    void *sampled, void *scratch, size_t scratch_bytes, int dtype, void *stream) {
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "fps: dtype %d", dtype);
  TK3D_REQUIRE(B >= 0 && N >= 0, TK3D_ERR_SHAPE, "fps: negative size");
  TK3D_REQUIRE(S > 0, TK3D_ERR_K, "fps: num_samples must be positive (got %lld)", (long long)S);
  TK3D_REQUIRE(N >= S, TK3D_ERR_K, "fps: num_samples %lld exceeds the %lld points of a cloud", (long long)S,
               (long long)N);
  TK3D_REQUIRE(N < (1LL << 31), TK3D_ERR_SHAPE, "fps: clouds limited to 2^31-1 points");
  TK3D_REQUIRE(B < (1LL << 31), TK3D_ERR_SHAPE, "fps: batch too large");
  if (B == 0) return TK3D_OK;
  TK3D_REQUIRE(points && index, TK3D_ERR_NULL, "fps: points/index is NULL");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t ps = channel_first ? 1 : 3, cs = channel_first ? N : 1;
  const size_t need = tk3d_fps_scratch_bytes(B, N, dtype);
  if (dtype == TK3D_F64 && N > 2048) {
    // a cluster of blocks per cloud (fps_cluster.cu): few clouds of 2049 to 8192 points, every cloud of
    // 8193 to 131072 points; no scratch.  Declines (false) what the kernels below do better.
    int rc = TK3D_OK;
    if (fps_cluster_f64((const double *)points, B, N, S, (int)ps, cs, index, (double *)sampled, st, &rc)) return rc;
  }
  if (need == 0 && dtype == TK3D_F64) {
    int threads = threads_for((N + 7) / 8);
    if (threads < 128) threads = 128;
    const int P = (int)((N + threads - 1) / threads);
    const size_t smem = (size_t)N * 24;
    const double *p = (const double *)points;
#define TK3D_FPS64_CASE(PP)                                                                                          \
  {                                                                                                                  \
    TK3D_CUDA(raise_smem_limit((const void *)fps_resident64_kernel<PP>, \
                                   (int)(FPS_RESIDENT64_MAX_N * 24)));                                               \
    fps_resident64_kernel<PP><<<(unsigned)B, threads, smem, st>>>(p, (int)N, (int)S, index, (int)ps, (int)cs,        \
                                                                  (double *)sampled);                                \
  }
    if (P <= 1) TK3D_FPS64_CASE(1)
    else if (P <= 2) TK3D_FPS64_CASE(2)
    else if (P <= 4) TK3D_FPS64_CASE(4)
    else TK3D_FPS64_CASE(8)
#undef TK3D_FPS64_CASE
    return check_launch("fps_resident64_kernel");
  }
  if (dtype == TK3D_F32 && N > 4096) {
    // a cluster of blocks per cloud (fps_cluster.cu): few clouds of 4097 to 16384 points, and every
    // cloud of 16385 to 262144 points; no scratch.  Declines (false) what the kernels below do better.
    int rc = TK3D_OK;
    if (fps_cluster_f32((const float *)points, B, N, S, (int)ps, cs, index, (float *)sampled, st, &rc)) return rc;
  }
  if (need == 0) {
    // Up to 8 points per thread in registers (16 with the coordinates left in shared memory); at
    // least 4 warps so that every SM sub-partition has work.
    int threads = threads_for((N + 7) / 8);
    if (threads < 128) threads = 128;
    const int P = (int)((N + threads - 1) / threads);
    const size_t smem = (size_t)N * 12;
    const float *p = (const float *)points;
#define TK3D_FPS_CASE(PP)                                                                                       \
  {                                                                                                             \
    TK3D_CUDA(raise_smem_limit((const void *)fps_resident_kernel<PP>, 98304)); \
    fps_resident_kernel<PP><<<(unsigned)B, threads, smem, st>>>(p, (int)N, (int)S, index, (int)ps, (int)cs,       \
                                                                (float *)sampled, 1.0f);                          \
  }
    if (P <= 2) TK3D_FPS_CASE(1)
    else if (P <= 4) TK3D_FPS_CASE(2)
    else if (P <= 8) TK3D_FPS_CASE(4)
    else {  // 8193..16384 points: 16 per thread, coordinates stay in shared memory (up to 192 KB)
      TK3D_CUDA(raise_smem_limit((const void *)fps_resident_kernel<8, false>, (int)(FPS_RESIDENT_MAX_N * 12)));
      fps_resident_kernel<8, false><<<(unsigned)B, threads, smem, st>>>(p, (int)N, (int)S, index, (int)ps, (int)cs,
                                                                        (float *)sampled, 1.0f);
    }
#undef TK3D_FPS_CASE
    return check_launch("fps_resident_kernel");
  }
  TK3D_REQUIRE(scratch != nullptr && scratch_bytes >= need, TK3D_ERR_SCRATCH,
               "fps: scratch of %zu bytes required, %zu given", need, scratch ? scratch_bytes : (size_t)0);
  const int threads = threads_for(N);
  if (dtype == TK3D_F32)
    fps_streaming_kernel<float><<<(unsigned)B, threads, 0, st>>>((const float *)points, N, S, index, (float *)scratch,
                                                                ps, cs, (float *)sampled);
  else
    fps_streaming_kernel<double><<<(unsigned)B, threads, 0, st>>>((const double *)points, N, S, index,
                                                                 (double *)scratch, ps, cs, (double *)sampled);
  return check_launch("fps_streaming_kernel");
}

extern "C" int tk3d_fps(const void *points, int64_t B, int64_t N, int64_t S, int64_t *index, void *scratch,
                        size_t scratch_bytes, int dtype, void *stream) {
  TK3D_RANGE("tk3d_fps");
  return fps_impl(points, B, N, S, 0, index, nullptr, scratch, scratch_bytes, dtype, stream);
}

extern "C" int tk3d_fps_layout(const void *points, int64_t B, int64_t N, int64_t S, int xyz_channel_first,
                               int64_t *index, void *scratch, size_t scratch_bytes, int dtype, void *stream) {
  TK3D_RANGE("tk3d_fps_layout");
  return fps_impl(points, B, N, S, xyz_channel_first != 0, index, nullptr, scratch, scratch_bytes, dtype, stream);
}

extern "C" int tk3d_fps_gather(const void *points, int64_t B, int64_t N, int64_t S, int channel_first,
                               int64_t *index, void *sampled, void *scratch, size_t scratch_bytes, int dtype,
                               void *stream) {
  TK3D_RANGE("tk3d_fps_gather");
  TK3D_REQUIRE(sampled != nullptr || B * S == 0, TK3D_ERR_NULL, "fps_gather: sampled is NULL");
  return fps_impl(points, B, N, S, channel_first, index, sampled, scratch, scratch_bytes, dtype, stream);
}

// ---------------------------------------------------------------------------------------------
// Farthest point sampling for callers that cannot provide scratch memory.
//
// Some hosts of this library may not allocate device memory at the point where they sample: code
// running under a framework's "no allocation in this region" guard, a plugin whose memory budget
// was fixed at start-up, or a C caller that has no allocator at hand and does not want one
// cudaMalloc/cudaFree pair per call.  For them the running-minimum array of
// the streaming kernel lives in a fixed array inside the library image instead of a caller buffer.
//
// The array belongs to the device the library is loaded on (each GPU that loads the library
// carries its own copy until the process exits).  Host code must not hand the symbol itself to a
// kernel -- on the host it is only a stand-in -- so the device address is looked up once per
// device with cudaGetSymbolAddress and cached.
namespace tk3d {
namespace {

constexpr size_t FPS_STATIC_SCRATCH_BYTES = 8u << 20;  // 8 MiB: B*N <= 2,097,152 (fp32) / 1,048,576 (fp64)

static __device__ __align__(256) unsigned char g_fps_static_scratch[FPS_STATIC_SCRATCH_BYTES];

constexpr int FPS_MAX_DEVICES = 64;
void *g_fps_static_ptr[FPS_MAX_DEVICES] = {nullptr};

// Device address of the static scratch on the CURRENT device (looked up on first use).
int fps_static_scratch_ptr(void **out) {
  int dev = -1;
  TK3D_CUDA(cudaGetDevice(&dev));
  TK3D_REQUIRE(dev >= 0 && dev < FPS_MAX_DEVICES, TK3D_ERR_UNSUPPORTED, "fps_static_scratch: device id %d", dev);
  void *p = __atomic_load_n(&g_fps_static_ptr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    // Two threads racing here both obtain the same address; the store is idempotent.
    TK3D_CUDA(cudaGetSymbolAddress(&p, g_fps_static_scratch));
    TK3D_REQUIRE(p != nullptr, TK3D_ERR_CUDA, "fps_static_scratch: cudaGetSymbolAddress returned NULL");
    __atomic_store_n(&g_fps_static_ptr[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return TK3D_OK;
}

}  // namespace
}  // namespace tk3d

extern "C" size_t tk3d_fps_static_scratch_capacity(void) { return tk3d::FPS_STATIC_SCRATCH_BYTES; }

extern "C" int tk3d_fps_static_scratch(const void *points, int64_t B, int64_t N, int64_t S, int64_t *index,
                                       int dtype, void *stream) {
  TK3D_RANGE("tk3d_fps_static_scratch");
  TK3D_REQUIRE(dtype == TK3D_F32 || dtype == TK3D_F64, TK3D_ERR_DTYPE, "fps_static_scratch: dtype %d", dtype);
  TK3D_REQUIRE(B >= 0 && N >= 0, TK3D_ERR_SHAPE, "fps_static_scratch: negative size");
  TK3D_REQUIRE(S > 0, TK3D_ERR_K, "fps_static_scratch: num_samples must be positive (got %lld)", (long long)S);
  TK3D_REQUIRE(N >= S, TK3D_ERR_K, "fps_static_scratch: num_samples %lld exceeds the %lld points of a cloud",
               (long long)S, (long long)N);
  TK3D_REQUIRE(N < (1LL << 31) && B < (1LL << 31), TK3D_ERR_SHAPE, "fps_static_scratch: size too large");
  const size_t elem = dtype == TK3D_F64 ? 8 : 4;
  // B and N are below 2^31, so the product cannot overflow 64 bits.
  const size_t need = (size_t)B * (size_t)N * elem;
  TK3D_REQUIRE(need <= FPS_STATIC_SCRATCH_BYTES, TK3D_ERR_SCRATCH,
               "fps_static_scratch: B*N = %lld running minima need %zu bytes, the built-in scratch holds %zu "
               "(use tk3d_fps with a caller-provided buffer for larger problems)",
               (long long)(B * N), need, (size_t)FPS_STATIC_SCRATCH_BYTES);
  if (B == 0) return TK3D_OK;
  TK3D_REQUIRE(points && index, TK3D_ERR_NULL, "fps_static_scratch: points/index is NULL");
  void *scratch = nullptr;
  const int rc = fps_static_scratch_ptr(&scratch);
  if (rc != TK3D_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = threads_for(N);
  // The kernel overwrites every running minimum it reads in its first step, so what an earlier
  // call left in the array does not matter and nothing has to be cleared.
  if (dtype == TK3D_F32)
    fps_streaming_kernel<float><<<(unsigned)B, threads, 0, st>>>((const float *)points, N, S, index, (float *)scratch);
  else
    fps_streaming_kernel<double><<<(unsigned)B, threads, 0, st>>>((const double *)points, N, S, index,
                                                                 (double *)scratch);
  return check_launch("fps_streaming_kernel (static scratch)");
}

TK3D_BOUNDS_TU(fps)
