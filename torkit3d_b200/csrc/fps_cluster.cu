// Farthest point sampling on thread-block clusters: float32 clouds of 4097 to 262144 points, float64
// clouds of 2049 to 131072 points.
//
// The resident kernel of fps.cu keeps a cloud in the registers of ONE block: its step is a chain of
// two block barriers over 32 warps and two block reductions (0.69 us at 8192 points), it ends at
// 16384 points, and beyond that the streaming kernel re-reads the cloud and its running minima from
// L2 in every step (4 clouds of 65536 points: 19 us per step).  Here a cluster of 4, 8 or 16 small
// blocks shares a cloud: every block keeps a contiguous slice of the points and their running
// minima in registers (8 to 32 points per thread), and the step has no block or cluster barrier at
// all -- see fps_warpcast_kernel.  32 clouds of 8192 points, 1024 samples: 0.56 ms against 0.70 ms;
// 4 clouds of 65536 points, 2048 samples: 2.0 ms against 39.9 ms for the streaming kernel.
//
// Measured and dropped: the same clusters with 1024-thread blocks that reduce inside the block
// first (two block barriers) and exchange one candidate per block behind a cluster barrier per
// step -- 0.78 to 1.2 ms on the 32 x 8192 case for clusters of 2 to 16 blocks (the cluster barrier
// alone costs about 0.4 us), 2.7 ms on 4 x 65536.
//
// Arithmetic, tie rule and padding are those of fps_resident_kernel; the reference's kernel is
// torkit3d/csrc/cuda/sample_farthest_points_kernel.cu:33-103 (one block per cloud, any size).
#include <cooperative_groups.h>

#include "tk3d_common.cuh"

namespace cg = cooperative_groups;

namespace tk3d {

constexpr int FC_MAX_CL = 16;  // 8 is the portable cluster size; 16 needs an opt-in

// ---------------------------------------------------------------------------------------------
// No block or cluster barrier in the step.  Every WARP finds its own farthest point (two REDUX)
// and sends it -- 20 bytes: distance bits, index, coordinates -- straight into the shared memory of
// every block of the cluster with st.async, which also counts the bytes on an mbarrier of the
// receiving block.  A warp then waits on its own block's mbarrier until the candidates of all
// warps of the cluster have landed, and lane l looks at candidates l, l + 32, ...: two more REDUX
// pick the winner (highest distance, lowest index), the same in every warp.  The candidate slots
// and mbarriers are double buffered by the step's parity: a warp can send for step i+2 only after
// it has seen every warp's candidate of step i+1, which those warps send after they have read
// step i.  The fewer warps a cluster has the shorter the step (its floor is the exchange over
// distributed shared memory, about 0.45 us), hence up to 32 points per thread.  Every wait is
// limited (limit_ns: one second in regular calls); a warp that runs into the limit stops, the
// rest of its cloud's index row is set to -1, fw_expired_waits counts it, and every block still
// leaves through the final cluster barrier.
struct __align__(16) FwCandidate {
  unsigned bits;
  int idx;
  float x, y;
  float z;
  int pad[3];
};
constexpr unsigned FW_CAND_BYTES = 20;

__device__ __forceinline__ unsigned fw_smem(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned fw_mapa(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ unsigned fw_try_wait(unsigned bar, unsigned phase) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(phase)
      : "memory");
  return ok;
}
__device__ __forceinline__ unsigned long long fw_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Waits that ran into their limit since the library was loaded (per device); read by
// tk3d_fps_expired_waits().
__device__ unsigned int fw_expired_waits = 0;

// FW_REGS false (clouds beyond 131072 points): the coordinates stay in shared memory, which then
// holds FW_THREADS * 2 * FW_P2 points, and only the running minima live in registers.
template <int FW_THREADS, int FW_P2, int FW_SLOTS, bool FW_REGS = true>
__global__ void __launch_bounds__(FW_THREADS)
fps_warpcast_kernel(const float *__restrict__ points, int N, int NL, int S, int64_t *__restrict__ index, int ps, int cs,
                    float *__restrict__ sampled, float one, unsigned long long limit_ns, int drop_step) {
  cg::cluster_group cluster = cg::this_cluster();
  const int CL = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int cloud = blockIdx.x / CL;
  extern __shared__ float sxyz[];  // [3*NL]: this block's slice of the cloud
  __shared__ FwCandidate cand[2][FW_SLOTS];  // one slot per warp of the cluster
  __shared__ __align__(8) unsigned long long mbar[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int T = FW_THREADS, W = FW_THREADS / 32;
  const int nw = CL * W;           // warps of the cluster, at most FW_SLOTS
  const int gw = rank * W + warp;  // this warp's candidate slot
  const float *pts = points + (int64_t)cloud * N * 3;
  int64_t *out = index + (int64_t)cloud * S;
  const int base = rank * NL;
  const int nloc = max(0, min(NL, N - base));

  for (int e = tid; e < 3 * nloc; e += T) {
    const int j = e / 3, d = e - 3 * j;
    sxyz[e] = pts[(int64_t)(base + j) * ps + (int64_t)d * cs];
  }
  const unsigned bar0 = fw_smem(&mbar[0]), bar1 = fw_smem(&mbar[1]);
  const unsigned expect = (unsigned)nw * FW_CAND_BYTES;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // steps 1 and 2 use barrier 1 and barrier 0
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar1), "r"(expect) : "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar0), "r"(expect) : "memory");
  }
  __syncthreads();

  constexpr int FW_PREG = FW_REGS ? FW_P2 : 1;
  float2 px[FW_PREG], py[FW_PREG], pz[FW_PREG], md[FW_P2];
  const float qnan = __int_as_float(0x7fc00000), pinf = __int_as_float(0x7f800000);
  if constexpr (!FW_REGS) {
    // padding slots of the shared-memory copy: NaN coordinates keep their distance of 0
    for (int e = 3 * nloc + tid; e < 3 * T * 2 * FW_P2; e += T) sxyz[e] = qnan;
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < FW_P2; ++i) {
    const int j0 = (2 * i) * T + tid, j1 = (2 * i + 1) * T + tid;
    if constexpr (FW_REGS) {
      px[i].x = j0 < nloc ? sxyz[3 * j0 + 0] : qnan;
      py[i].x = j0 < nloc ? sxyz[3 * j0 + 1] : qnan;
      pz[i].x = j0 < nloc ? sxyz[3 * j0 + 2] : qnan;
      px[i].y = j1 < nloc ? sxyz[3 * j1 + 0] : qnan;
      py[i].y = j1 < nloc ? sxyz[3 * j1 + 1] : qnan;
      pz[i].y = j1 < nloc ? sxyz[3 * j1 + 2] : qnan;
    }
    md[i].x = j0 < nloc ? pinf : 0.f;
    md[i].y = j1 < nloc ? pinf : 0.f;
  }

  float cx = pts[0], cy = pts[cs], cz = pts[2 * (int64_t)cs];
  const bool writer = rank == 0 && tid == 0;
  const int sps = cs == 1 ? 3 : 1, scs = cs == 1 ? 1 : S;
  float *sm = sampled ? sampled + (int64_t)cloud * S * 3 : nullptr;
  if (writer) {
    out[0] = 0;
    if (sm) {
      sm[0] = cx;
      sm[scs] = cy;
      sm[2 * (int64_t)scs] = cz;
    }
  }
  cluster.sync();  // every block's mbarriers are initialised and armed: candidates may be sent

  // this lane's target block when it sends (lanes 0..CL-1 of every warp)
  const unsigned tgt = (unsigned)(lane < CL ? lane : 0);
  const unsigned rcand0 = fw_mapa(fw_smem(&cand[0][gw]), tgt), rcand1 = fw_mapa(fw_smem(&cand[1][gw]), tgt);
  const unsigned rbar0 = fw_mapa(bar0, tgt), rbar1 = fw_mapa(bar1, tgt);

  const float2 one2 = make_float2(one, one);
  bool failed = false;
  int it = 1;
  for (; it < S; ++it) {
    const int par = it & 1;
    const float2 ncx = make_float2(-cx, -cx), ncy = make_float2(-cy, -cy), ncz = make_float2(-cz, -cz);
    float bm = 0.f;
#pragma unroll
    for (int i = 0; i < FW_P2; ++i) {
      float2 qx_, qy_, qz_;
      if constexpr (FW_REGS) {
        qx_ = px[i];
        qy_ = py[i];
        qz_ = pz[i];
      } else {
        const float *a0 = sxyz + 3 * ((2 * i) * T + tid), *a1 = sxyz + 3 * ((2 * i + 1) * T + tid);
        qx_ = make_float2(a0[0], a1[0]);
        qy_ = make_float2(a0[1], a1[1]);
        qz_ = make_float2(a0[2], a1[2]);
      }
      const float2 dx = __fadd2_rn(qx_, ncx), dy = __fadd2_rn(qy_, ncy), dz = __fadd2_rn(qz_, ncz);
      const float2 d = __ffma2_rn(__ffma2_rn(__fmul2_rn(dx, dx), one2, __fmul2_rn(dy, dy)), one2, __fmul2_rn(dz, dz));
      md[i].x = fminf(md[i].x, d.x);
      md[i].y = fminf(md[i].y, d.y);
      asm("max.f32 %0, %0, %1, %2;" : "+f"(bm) : "f"(md[i].x), "f"(md[i].y));
    }
    const unsigned bits = __float_as_uint(bm);
    const unsigned gb = __reduce_max_sync(0xffffffffu, bits);
    int mine = 0x7fffffff;
    if (bits == gb) {
#pragma unroll
      for (int i = FW_P2 - 1; i >= 0; --i) {
        if (md[i].y == bm) mine = (2 * i + 1) * T + tid;
        if (md[i].x == bm) mine = (2 * i) * T + tid;
      }
    }
    const int loc = __reduce_min_sync(0xffffffffu, mine);  // lowest local index holding the warp's maximum
    if (lane < CL && !(it == drop_step && gw == 0)) {  // drop_step: diagnostic only, -1 otherwise
      const bool real = loc < nloc;
      const float x = real ? sxyz[3 * loc + 0] : 0.f, y = real ? sxyz[3 * loc + 1] : 0.f,
                  z = real ? sxyz[3 * loc + 2] : 0.f;
      const unsigned rc = par ? rcand1 : rcand0, rb = par ? rbar1 : rbar0;
      asm volatile(
          "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(rc),
          "r"(gb), "r"(base + loc), "r"(__float_as_uint(x)), "r"(__float_as_uint(y)), "r"(rb)
          : "memory");
      asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(rc + 16),
                   "r"(__float_as_uint(z)), "r"(rb)
                   : "memory");
    }
    // wait until the candidates of all warps of the cluster have landed in this block
    const unsigned lb = par ? bar1 : bar0, phase = (unsigned)((it - 1) >> 1) & 1u;
    unsigned ok = fw_try_wait(lb, phase);
    if (!ok) {  // bounded by time (limit_ns: one second) and by count
      const unsigned long long t0 = fw_now();
      for (int spin = 0; spin < (1 << 24) && !ok; ++spin) {
        ok = fw_try_wait(lb, phase);
        if (!ok && fw_now() - t0 > limit_ns) break;
      }
    }
    if (!__all_sync(0xffffffffu, ok != 0)) {
      failed = true;
      break;
    }
    // the barrier just completed is used again two steps on
    if (tid == 0 && it + 2 < S)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(lb), "r"(expect) : "memory");
    // lane l looks at candidates l, l + 32, ...: highest distance, then lowest index
    const bool has = lane < nw;
    unsigned cb = 0u;
    int ci = 0x7fffffff, slot = lane;
    if constexpr (FW_SLOTS <= 32) {
      cb = has ? cand[par][lane].bits : 0u;
      ci = has ? cand[par][lane].idx : 0x7fffffff;
    } else {
      for (int sl = lane; sl < nw; sl += 32) {
        const unsigned b_ = cand[par][sl].bits;
        const int i_ = cand[par][sl].idx;
        if (b_ > cb || (b_ == cb && i_ < ci)) {
          cb = b_;
          ci = i_;
          slot = sl;
        }
      }
    }
    const unsigned wb = __reduce_max_sync(0xffffffffu, cb);
    const int wi = __reduce_min_sync(0xffffffffu, (has && cb == wb) ? ci : 0x7fffffff);
    int src = __ffs(__ballot_sync(0xffffffffu, has && cb == wb && ci == wi)) - 1;
    if constexpr (FW_SLOTS > 32) src = __shfl_sync(0xffffffffu, slot, src);
    cx = cand[par][src].x;
    cy = cand[par][src].y;
    cz = cand[par][src].z;
    if (writer) {
      out[it] = wi;
      if (sm) {
        sm[(int64_t)it * sps] = cx;
        sm[(int64_t)it * sps + scs] = cy;
        sm[(int64_t)it * sps + 2 * (int64_t)scs] = cz;
      }
    }
  }
  if (failed && lane == 0) atomicAdd(&fw_expired_waits, 1u);
  if (failed && rank == 0 && warp == 0 && lane == 0)
    for (int r = it; r < S; ++r) out[r] = -1;  // a wait ran into its limit: the rest of the row is marked
  cluster.sync();  // no block leaves while a candidate may still be on its way into its shared memory
}

// ---------------------------------------------------------------------------------------------
// float64: the same step on doubles.  The coordinates stay in the block's shared-memory copy (24
// bytes per point), the running minima live in registers (P per thread); a candidate is 40 bytes
// (64-bit distance pattern, index, three doubles), the maxima are taken on the 64-bit pattern in
// two REDUX steps.  Arithmetic as in fps_resident64_kernel: ((dx*dx + dy*dy) + dz*dz) with
// individually rounded operations.
struct __align__(16) FwCandidate64 {
  unsigned long long bits;
  int idx;
  int pad;
  double x, y;
  double z;
  double pad2;
};
constexpr unsigned FW_CAND64_BYTES = 40;

__device__ __forceinline__ unsigned long long fw_warp_max64(unsigned long long v) {
  const unsigned hi = (unsigned)(v >> 32), lo = (unsigned)v;
  const unsigned whi = __reduce_max_sync(0xffffffffu, hi);
  const unsigned wlo = __reduce_max_sync(0xffffffffu, hi == whi ? lo : 0u);
  return ((unsigned long long)whi << 32) | wlo;
}

template <int FW_THREADS, int FW_P, int FW_SLOTS>
__global__ void __launch_bounds__(FW_THREADS)
fps_warpcast64_kernel(const double *__restrict__ points, int N, int NL, int S, int64_t *__restrict__ index, int ps,
                      int cs, double *__restrict__ sampled, unsigned long long limit_ns, int drop_step) {
  cg::cluster_group cluster = cg::this_cluster();
  const int CL = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int cloud = blockIdx.x / CL;
  extern __shared__ double dxyz[];  // [3 * FW_THREADS * FW_P]: this block's slice, padded with NaN
  __shared__ FwCandidate64 cand[2][FW_SLOTS];
  __shared__ __align__(8) unsigned long long mbar[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int T = FW_THREADS, W = FW_THREADS / 32;
  const int nw = CL * W, gw = rank * W + warp;
  const double *pts = points + (int64_t)cloud * N * 3;
  int64_t *out = index + (int64_t)cloud * S;
  const int base = rank * NL;
  const int nloc = max(0, min(NL, N - base));
  const double qnan = __longlong_as_double(0x7ff8000000000000LL);

  for (int e = tid; e < 3 * T * FW_P; e += T) {
    const int j = e / 3, d = e - 3 * j;
    dxyz[e] = j < nloc ? pts[(int64_t)(base + j) * ps + (int64_t)d * cs] : qnan;
  }
  const unsigned bar0 = fw_smem(&mbar[0]), bar1 = fw_smem(&mbar[1]);
  const unsigned expect = (unsigned)nw * FW_CAND64_BYTES;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar1), "r"(expect) : "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar0), "r"(expect) : "memory");
  }
  __syncthreads();

  // Point i of this thread is local j = i * T + tid; padding keeps a running minimum of 0.
  double md[FW_P];
#pragma unroll
  for (int i = 0; i < FW_P; ++i) md[i] = (i * T + tid) < nloc ? Exact<double>::inf() : 0.0;

  double cx = pts[0], cy = pts[cs], cz = pts[2 * (int64_t)cs];
  const bool writer = rank == 0 && tid == 0;
  const int sps = cs == 1 ? 3 : 1, scs = cs == 1 ? 1 : S;
  double *sm = sampled ? sampled + (int64_t)cloud * S * 3 : nullptr;
  if (writer) {
    out[0] = 0;
    if (sm) {
      sm[0] = cx;
      sm[scs] = cy;
      sm[2 * (int64_t)scs] = cz;
    }
  }
  cluster.sync();

  const unsigned tgt = (unsigned)(lane < CL ? lane : 0);
  const unsigned rcand0 = fw_mapa(fw_smem(&cand[0][gw]), tgt), rcand1 = fw_mapa(fw_smem(&cand[1][gw]), tgt);
  const unsigned rbar0 = fw_mapa(bar0, tgt), rbar1 = fw_mapa(bar1, tgt);

  bool failed = false;
  int it = 1;
  for (; it < S; ++it) {
    const int par = it & 1;
    double bm = 0.0;
#pragma unroll
    for (int i = 0; i < FW_P; ++i) {
      const double *a = dxyz + 3 * (i * T + tid);
      const double d = sqdist<double>(a[0], a[1], a[2], cx, cy, cz);
      md[i] = fmin(md[i], d);
      bm = fmax(bm, md[i]);
    }
    const unsigned long long bits = (unsigned long long)__double_as_longlong(bm);
    const unsigned long long gb = fw_warp_max64(bits);
    int mine = 0x7fffffff;
    if (bits == gb) {
#pragma unroll
      for (int i = FW_P - 1; i >= 0; --i)
        if (md[i] == bm) mine = i * T + tid;
    }
    const int loc = __reduce_min_sync(0xffffffffu, mine);
    if (lane < CL && !(it == drop_step && gw == 0)) {
      const bool real = loc < nloc;
      const double x = real ? dxyz[3 * loc + 0] : 0.0, y = real ? dxyz[3 * loc + 1] : 0.0,
                   z = real ? dxyz[3 * loc + 2] : 0.0;
      const unsigned rc = par ? rcand1 : rcand0, rb = par ? rbar1 : rbar0;
      asm volatile(
          "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(rc),
          "r"((unsigned)gb), "r"((unsigned)(gb >> 32)), "r"(base + loc), "r"(0), "r"(rb)
          : "memory");
      asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b64 [%0], {%1, %2}, [%3];" ::"r"(rc + 16),
                   "l"(__double_as_longlong(x)), "l"(__double_as_longlong(y)), "r"(rb)
                   : "memory");
      asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b64 [%0], %1, [%2];" ::"r"(rc + 32),
                   "l"(__double_as_longlong(z)), "r"(rb)
                   : "memory");
    }
    const unsigned lb = par ? bar1 : bar0, phase = (unsigned)((it - 1) >> 1) & 1u;
    unsigned ok = fw_try_wait(lb, phase);
    if (!ok) {
      const unsigned long long t0 = fw_now();
      for (int spin = 0; spin < (1 << 24) && !ok; ++spin) {
        ok = fw_try_wait(lb, phase);
        if (!ok && fw_now() - t0 > limit_ns) break;
      }
    }
    if (!__all_sync(0xffffffffu, ok != 0)) {
      failed = true;
      break;
    }
    if (tid == 0 && it + 2 < S)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(lb), "r"(expect) : "memory");
    const bool has = lane < nw;
    unsigned long long cb = 0ull;
    int ci = 0x7fffffff, slot = lane;
    for (int sl = lane; sl < nw; sl += 32) {
      const unsigned long long b_ = cand[par][sl].bits;
      const int i_ = cand[par][sl].idx;
      if (b_ > cb || (b_ == cb && i_ < ci)) {
        cb = b_;
        ci = i_;
        slot = sl;
      }
    }
    const unsigned long long wb = fw_warp_max64(has ? cb : 0ull);
    const int wi = __reduce_min_sync(0xffffffffu, (has && cb == wb) ? ci : 0x7fffffff);
    int src = __ffs(__ballot_sync(0xffffffffu, has && cb == wb && ci == wi)) - 1;
    src = __shfl_sync(0xffffffffu, slot, src);
    cx = cand[par][src].x;
    cy = cand[par][src].y;
    cz = cand[par][src].z;
    if (writer) {
      out[it] = wi;
      if (sm) {
        sm[(int64_t)it * sps] = cx;
        sm[(int64_t)it * sps + scs] = cy;
        sm[(int64_t)it * sps + 2 * (int64_t)scs] = cz;
      }
    }
  }
  if (failed && lane == 0) atomicAdd(&fw_expired_waits, 1u);
  if (failed && rank == 0 && warp == 0 && lane == 0)
    for (int r = it; r < S; ++r) out[r] = -1;
  cluster.sync();
}

struct FwWait {
  unsigned long long limit_ns;  // every wait for the other warps' candidates gives up after this long
  int drop_step;                // diagnostic: the step in which one warp per cluster sends nothing; -1: none
};

// Cluster launch shared by the float32 and float64 kernels; `args` are the kernel's arguments.
static bool fps_cluster_launch_any(const void *kern, int THREADS, int64_t B, size_t smem, size_t smem_limit,
                                   cudaStream_t st, int *rc, int CL, void **args) {
  if (raise_smem_limit(kern, (int)smem_limit) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  if (CL > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(B * CL));
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelExC(&cfg, kern, args);
  if (e != cudaSuccess) {  // e.g. a device partition without room for the cluster
    (void)cudaGetLastError();
    return false;
  }
  *rc = check_launch("fps_warpcast_kernel");
  return true;
}

using FpsClusterKernel = void (*)(const float *, int, int, int, int64_t *, int, int, float *, float,
                                  unsigned long long, int);

static bool fps_cluster_launch_kernel(FpsClusterKernel kern, int THREADS, const float *points, int64_t B, int64_t N,
                                      int64_t S, int ps, int64_t cs, int64_t *index, float *sampled, cudaStream_t st,
                                      int *rc, int CL, FwWait wt, size_t smem_fixed = 0) {
  int n = (int)N, NL = (int)((N + CL - 1) / CL), s_ = (int)S, cs_ = (int)cs;
  float one = 1.0f;
  const size_t smem = smem_fixed ? smem_fixed : (size_t)NL * 12;
  void *args[] = {&points, &n, &NL, &s_, &index, &ps, &cs_, &sampled, &one, &wt.limit_ns, &wt.drop_step};
  return fps_cluster_launch_any((const void *)kern, THREADS, B, smem, smem_fixed ? smem_fixed : 98304, st, rc, CL, args);
}

template <int THREADS, int P, int SLOTS>
static bool fps_warpcast64_launch(const double *points, int64_t B, int64_t N, int64_t S, int ps, int64_t cs,
                                  int64_t *index, double *sampled, cudaStream_t st, int *rc, int CL, FwWait wt) {
  if (CL * (THREADS / 32) > SLOTS || (int64_t)CL * THREADS * P < N) return false;  // a slot per warp, a register per point
  int n = (int)N, NL = (int)((N + CL - 1) / CL), s_ = (int)S, cs_ = (int)cs;
  const size_t smem = (size_t)THREADS * P * 24;
  void *args[] = {&points, &n, &NL, &s_, &index, &ps, &cs_, &sampled, &wt.limit_ns, &wt.drop_step};
  return fps_cluster_launch_any((const void *)fps_warpcast64_kernel<THREADS, P, SLOTS>, THREADS, B, smem, smem, st, rc,
                                CL, args);
}

template <int THREADS, int P2>
static bool fps_warpcast_launch(const float *points, int64_t B, int64_t N, int64_t S, int ps, int64_t cs, int64_t *index,
                                float *sampled, cudaStream_t st, int *rc, int CL, FwWait wt) {
  if (CL * (THREADS / 32) > 512 || (int64_t)CL * THREADS * 2 * P2 < N) return false;  // a slot per warp, a register per point
  if (CL * (THREADS / 32) <= 32)
    return fps_cluster_launch_kernel(fps_warpcast_kernel<THREADS, P2, 32>, THREADS, points, B, N, S, ps, cs, index,
                                     sampled, st, rc, CL, wt);
  return fps_cluster_launch_kernel(fps_warpcast_kernel<THREADS, P2, 512>, THREADS, points, B, N, S, ps, cs, index,
                                   sampled, st, rc, CL, wt);
}

// Launches a cluster kernel when the clouds suit one (float32, 4096 < N <= 262144); returns false
// when they do not or when the device refuses the cluster launch (the caller then takes its own
// path), true with *rc set otherwise.
//
// 4097 to 16384 points and few clouds: up to 8192 points clusters of four blocks of 256 threads (8
// points per thread), beyond that eight blocks of 128 threads (16 points per thread).  Measured on
// two B200s, 512 samples, against one 1024-thread block per cloud (fps_resident_kernel), in ms:
//   clouds                      4      32     64     96
//   N =  8192  4 x 256 threads  0.26-0.27  0.28  0.33   0.40     one block  0.356
//              8 x  64 threads  0.25-0.29  0.27-0.31  0.30-0.33  0.36   (faster on one GPU, slower on the other)
//   N = 16384  8 x 128 threads  0.30   0.34-0.37  0.45   0.76     one block  0.699
// Beyond about half a cloud per SM the blocks of several clusters share SMs and the one-block
// kernel is as fast; up to 4096 points its step (0.43 us) is shorter than the exchange over
// distributed shared memory (0.45 to 0.5 us).
static bool fps_cluster_dispatch(const float *points, int64_t B, int64_t N, int64_t S, int ps, int64_t cs,
                                 int64_t *index, float *sampled, cudaStream_t st, int *rc, FwWait wt, bool force) {
  if (N > 4096 && N <= 16384) {
    if (N <= 8192) {
      if (!force && B * 15 > (int64_t)sm_count() * 7) return false;
      return fps_warpcast_launch<256, 4>(points, B, N, S, ps, cs, index, sampled, st, rc, 4, wt);
    }
    if (!force && B * 15 > (int64_t)sm_count() * 8) return false;
    return fps_warpcast_launch<128, 8>(points, B, N, S, ps, cs, index, sampled, st, rc, 8, wt);
  }
  if (N <= 16384 || N > 262144 || B * FC_MAX_CL >= (1LL << 31)) return false;
  if (N > 131072)  // 64 points per thread: running minima in registers, coordinates in 192 KB of shared memory
    return fps_cluster_launch_kernel(fps_warpcast_kernel<256, 32, 128, false>, 256, points, B, N, S, ps, cs, index,
                                     sampled, st, rc, 16, wt, (size_t)256 * 64 * 12);
  // larger clouds: 32 points per thread, so that a cluster has at most 128 warps (4 clouds, 512 samples:
  // 32768 points 0.375 ms, 0.48 with 16 points per thread and twice the warps; 65536 points 0.51 / 0.60)
  if (N <= 32768) return fps_warpcast_launch<128, 16>(points, B, N, S, ps, cs, index, sampled, st, rc, 8, wt);
  if (N <= 65536) return fps_warpcast_launch<128, 16>(points, B, N, S, ps, cs, index, sampled, st, rc, 16, wt);
  return fps_warpcast_launch<256, 16>(points, B, N, S, ps, cs, index, sampled, st, rc, 16, wt);
}

// float64: few clouds of 2049 to 8192 points (the one-block kernel's step is 1.1 us at 4096 points),
// every cloud of 8193 to 131072 points (the streaming kernel otherwise).
bool fps_cluster_f64(const double *points, int64_t B, int64_t N, int64_t S, int ps, int64_t cs, int64_t *index,
                     double *sampled, cudaStream_t st, int *rc) {
  const FwWait wt{1000000000ull, -1};
  if (N <= 2048 || N > 131072 || B * FC_MAX_CL >= (1LL << 31)) return false;
  // Double-precision arithmetic makes the distance updates the longer part of the step, so the
  // clouds are spread over more threads than in float32 (4 to 32 points per thread).  Measured, 256
  // samples of 4 / 32 clouds, in ms: 4096 points 0.20 / 0.23 (one block per cloud 0.29), 8192 points
  // 0.26 / 0.32 (0.46), 16384 points 0.29 / 0.38 (streaming kernel 2.2), 65536 points 0.57 / 1.8 (6.6).
  if (N <= 8192) {
    if (B * 15 > (int64_t)sm_count() * 8) return false;
    if (N <= 4096) return fps_warpcast64_launch<128, 4, 32>(points, B, N, S, ps, cs, index, sampled, st, rc, 8, wt);
    return fps_warpcast64_launch<256, 4, 128>(points, B, N, S, ps, cs, index, sampled, st, rc, 8, wt);
  }
  if (N <= 16384) return fps_warpcast64_launch<256, 8, 128>(points, B, N, S, ps, cs, index, sampled, st, rc, 8, wt);
  if (N <= 32768) return fps_warpcast64_launch<256, 16, 128>(points, B, N, S, ps, cs, index, sampled, st, rc, 8, wt);
  if (N <= 65536) return fps_warpcast64_launch<256, 16, 128>(points, B, N, S, ps, cs, index, sampled, st, rc, 16, wt);
  return fps_warpcast64_launch<256, 32, 128>(points, B, N, S, ps, cs, index, sampled, st, rc, 16, wt);
}

bool fps_cluster_f32(const float *points, int64_t B, int64_t N, int64_t S, int ps, int64_t cs, int64_t *index,
                     float *sampled, cudaStream_t st, int *rc) {
  return fps_cluster_dispatch(points, B, N, S, ps, cs, index, sampled, st, rc, FwWait{1000000000ull, -1}, false);
}

}  // namespace tk3d

using namespace tk3d;

extern "C" long long tk3d_fps_expired_waits(void) {
  unsigned int v = 0;
  if (cudaMemcpyFromSymbol(&v, fw_expired_waits, sizeof(v)) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  return (long long)v;
}

extern "C" int tk3d_diag_fps_wait_limit(const void *points, int64_t B, int64_t N, int64_t num_samples, int64_t *index,
                                        int64_t limit_ms, int64_t drop_step, void *stream) {
  TK3D_REQUIRE(points && index, TK3D_ERR_NULL, "diag_fps_wait_limit: a pointer is NULL");
  TK3D_REQUIRE(B > 0 && N > 4096 && N <= 131072 && num_samples > 0 && num_samples <= N, TK3D_ERR_SHAPE,
               "diag_fps_wait_limit: needs 4096 < N <= 131072 and 0 < num_samples <= N");
  TK3D_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, TK3D_ERR_SHAPE, "diag_fps_wait_limit: limit of 1 to 1000 ms");
  int rc = TK3D_OK;
  const FwWait wt{(unsigned long long)limit_ms * 1000000ull, (int)drop_step};
  if (!fps_cluster_dispatch((const float *)points, B, N, num_samples, 3, 1, index, nullptr, (cudaStream_t)stream, &rc, wt,
                            true))
    return fail(TK3D_ERR_CUDA, "diag_fps_wait_limit: the device refused the cluster launch");
  return rc;
}

TK3D_BOUNDS_TU(fps_cluster)
