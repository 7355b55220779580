// Version, error strings and per-thread error messages of libtk3d_b200.
#include <stdarg.h>
#include <string.h>

#include <mutex>

#include <nvtx3/nvToolsExt.h>

#include "tk3d_common.cuh"

namespace tk3d {

static thread_local char g_err[512] = "";

char *last_error_buffer() { return g_err; }

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int sm_count() {
  // One slot per device id; a benign race only ever stores the same value twice.
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes), issued only when
// this (kernel, device) pair has not been given at least `bytes` yet.  The attribute sticks to the
// function for the life of the context, and re-issuing it on every call costs host time that the
// small, launch-bound operators notice.  A fixed table with a mutex: a few dozen kernels exist.
cudaError_t raise_smem_limit(const void *func, int bytes) {
  struct Entry {
    const void *func;
    int dev;
    int bytes;
  };
  constexpr int CAP = 256;
  static Entry table[CAP];
  static int used = 0;
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  Entry *slot = nullptr;
  for (int i = 0; i < used; ++i)
    if (table[i].func == func && table[i].dev == dev) {
      slot = &table[i];
      break;
    }
  if (slot && slot->bytes >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return e;
  if (!slot && used < CAP) {
    slot = &table[used++];
    slot->func = func;
    slot->dev = dev;
    slot->bytes = 0;
  }
  if (slot) slot->bytes = bytes;
  return cudaSuccess;
}

void nvtx_push(const char *name) { nvtxRangePushA(name); }
void nvtx_pop() { nvtxRangePop(); }

}  // namespace tk3d

extern "C" {

int tk3d_version(void) { return 100; }

const char *tk3d_strerror(int code) {
  switch (code) {
    case TK3D_OK: return "ok";
    case TK3D_ERR_NULL: return "a required pointer is NULL";
    case TK3D_ERR_SHAPE: return "invalid tensor size";
    case TK3D_ERR_K: return "k / num_samples out of range";
    case TK3D_ERR_DTYPE: return "unsupported dtype";
    case TK3D_ERR_CUDA: return "CUDA error";
    case TK3D_ERR_SCRATCH: return "scratch buffer missing or too small";
    case TK3D_ERR_UNSUPPORTED: return "unsupported request";
    default: return "unknown error code";
  }
}

const char *tk3d_last_error(void) { return tk3d::last_error_buffer(); }

#ifdef TK3D_BOUNDS
unsigned long long tk3d_bounds_count_ball_query(void);
unsigned long long tk3d_bounds_count_chamfer(void);
unsigned long long tk3d_bounds_count_chamfer_fast(void);
unsigned long long tk3d_bounds_count_diag(void);
unsigned long long tk3d_bounds_count_edge(void);
unsigned long long tk3d_bounds_count_feature_knn(void);
unsigned long long tk3d_bounds_count_fps(void);
unsigned long long tk3d_bounds_count_fps_cluster(void);
unsigned long long tk3d_bounds_count_group(void);
unsigned long long tk3d_bounds_count_interp(void);
unsigned long long tk3d_bounds_count_knn(void);
unsigned long long tk3d_bounds_count_knn_select(void);
unsigned long long tk3d_bounds_count_knn_split(void);
unsigned long long tk3d_bounds_count_sa_group(void);
#endif

long long tk3d_bounds_violations(void) {
#ifdef TK3D_BOUNDS
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  return (long long)(tk3d_bounds_count_ball_query() + tk3d_bounds_count_chamfer() + tk3d_bounds_count_chamfer_fast() + tk3d_bounds_count_diag() + tk3d_bounds_count_edge() + tk3d_bounds_count_feature_knn() + tk3d_bounds_count_fps() + tk3d_bounds_count_fps_cluster() + tk3d_bounds_count_group() + tk3d_bounds_count_interp() + tk3d_bounds_count_knn() + tk3d_bounds_count_knn_select() + tk3d_bounds_count_knn_split() + tk3d_bounds_count_sa_group());
#else
  return -1;  // this build carries no range checks
#endif
}

}  // extern "C"
