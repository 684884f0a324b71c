// Norm backward that allocates nothing: its scratch is a file-scope device array.
// See norm_noalloc.h for who needs this and for the limits.
#include "norm_noalloc.h"

#include "../common/host.h"

namespace zb {
int norm_bwd_with_scratch(const void* dy, const void* x, const void* w, const float* stats, const void* dres, void* dx,
                          float* part_dw, float* part_db, int P, void* dw, void* db, int T, int H, int ln, int grad_f32,
                          int accumulate, cudaStream_t stream);
}

// Two planes (weight-gradient partials, bias-gradient partials) of ROWS x MAX_H floats.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) float g_norm_scratch[2 * ZB_NORM_NOALLOC_ROWS * ZB_NORM_NOALLOC_MAX_H];

static float* scratch_for_current_device(int* err) {
  static float* cached[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *err = -2;
    snprintf(zb::last_error_buf(), 512, "norm_bwd_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    return nullptr;
  }
  if (cached[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_norm_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *err = -2;
      snprintf(zb::last_error_buf(), 512, "norm_bwd_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cached[dev] = p;
  }
  return cached[dev];
}

extern "C" int zb_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* stats, const void* dres,
                                   void* dx, void* dw, void* db, int T, int H, int ln, int grad_f32, int accumulate,
                                   cudaStream_t stream) {
  if (H % 8 != 0 || H <= 0)
    ZB_FAIL(-1, "norm_bwd_noalloc: H=%d must be a positive multiple of 8", H);
  if (H > ZB_NORM_NOALLOC_MAX_H)
    ZB_FAIL(-1, "norm_bwd_noalloc: H=%d exceeds the built-in scratch (max %d); use zb_norm_bwd with caller scratch",
            H, ZB_NORM_NOALLOC_MAX_H);
  if (T <= 0) return 0;
  int err = 0;
  float* scratch = scratch_for_current_device(&err);
  if (scratch == nullptr) return err;
  const int P = T < ZB_NORM_NOALLOC_ROWS ? T : ZB_NORM_NOALLOC_ROWS;
  float* part_dw = scratch;
  float* part_db = scratch + size_t(ZB_NORM_NOALLOC_ROWS) * ZB_NORM_NOALLOC_MAX_H;
  // rows [0, P) x [0, H) of each plane are fully rewritten by the first kernel before the
  // second one reads them, so stale contents of earlier calls never leak into the result
  return zb::norm_bwd_with_scratch(dy, x, w, stats, dres, dx, part_dw, part_db, P, dw, db, T, H, ln, grad_f32,
                                   accumulate, stream);
}

extern "C" int zb_norm_bwd_noalloc_init(void) {
  int err = 0;
  return scratch_for_current_device(&err) != nullptr ? 0 : err;
}
