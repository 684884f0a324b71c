// Host-side helpers shared by every launcher: TMA tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), device attributes, and the
// error-return convention (0 = ok, negative = host-side failure, see zb_last_error()).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

namespace zb {

inline char* last_error_buf() {
  static thread_local char buf[512];
  return buf;
}
#define ZB_FAIL(code, ...)                                   \
  do {                                                       \
    snprintf(zb::last_error_buf(), 512, __VA_ARGS__);        \
    return (code);                                           \
  } while (0)
#define ZB_CUDA_OK(expr)                                                              \
  do {                                                                                \
    cudaError_t e_ = (expr);                                                          \
    if (e_ != cudaSuccess) ZB_FAIL(-2, "%s: %s", #expr, cudaGetErrorString(e_));      \
  } while (0)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor, row-major: `rows` x `cols`, row stride `ld` elements; box = box_cols x
// box_rows with 128-byte swizzle (box_cols must be 64). Returns 0 on success.
inline int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                             uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) ZB_FAIL(-3, "cuTensorMapEncodeTiled entry point not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) ZB_FAIL(-4, "TMA base not 16-byte aligned");
  if ((ld * 2) % 16 != 0) ZB_FAIL(-4, "TMA row stride (%llu elements) not a multiple of 16 bytes",
                                  (unsigned long long)ld);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) ZB_FAIL(-5, "cuTensorMapEncodeTiled failed with %d", int(r));
  return 0;
}

// General N-d bf16 tensor map (innermost dimension first), 128-byte swizzle.
inline int make_tmap_nd_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                             const uint64_t* strides_bytes /* rank-1 */, const uint32_t* box) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) ZB_FAIL(-3, "cuTensorMapEncodeTiled entry point not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) ZB_FAIL(-4, "TMA base not 16-byte aligned");
  cuuint64_t d[5];
  cuuint64_t s[4];
  cuuint32_t b[5], e[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    e[i] = 1;
    if (i < rank - 1) {
      s[i] = strides_bytes[i];
      if (s[i] % 16 != 0) ZB_FAIL(-4, "TMA stride %d not a multiple of 16 bytes", i);
    }
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), d, s, b, e,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) ZB_FAIL(-5, "cuTensorMapEncodeTiled failed with %d", int(r));
  return 0;
}

inline int num_sms() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (n[dev] == 0) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev] > 0 ? n[dev] : 148;
}

}  // namespace zb
