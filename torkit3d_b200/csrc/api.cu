// Version, error strings and per-thread error messages of libtk3d_b200.
#include <stdarg.h>
#include <string.h>

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

}  // extern "C"
