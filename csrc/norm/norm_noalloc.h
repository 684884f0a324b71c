// Allocation-free variant of the RMSNorm / LayerNorm backward.
//
// This entry point has no counterpart in the reference framework.  It exists for callers
// that must not allocate device memory while they run: code executing inside a memory-pool
// or allocator callback, a host thread that is not allowed to take the allocator's lock, a
// plugin that lives in a process whose memory budget is owned by someone else.  The regular
// entry point `zb_norm_bwd` needs two fp32 scratch planes (per-CTA partial sums of the weight
// and bias gradients) that its caller allocates; here that scratch is a fixed array compiled
// into the library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch: hidden size H <= ZB_NORM_NOALLOC_MAX_H. The scratch is
// 2 planes x ZB_NORM_NOALLOC_ROWS x ZB_NORM_NOALLOC_MAX_H floats = 8 MiB of device memory on
// every GPU that loads the library, held until the process exits.
#define ZB_NORM_NOALLOC_MAX_H 8192
#define ZB_NORM_NOALLOC_ROWS 128

// Same arguments and results as zb_norm_bwd minus the two scratch pointers:
//   dx = (dres +) d(norm)/dx,  dw / db (+)= weight / bias gradients (fp32 if grad_f32 else bf16).
// Returns 0 on success; -1 with a message in zb_last_error() if H exceeds the limit or is not a
// multiple of 8; -2 on a CUDA error.
//
// * Calls no cudaMalloc / cudaFree and no allocating library routine.
// * The first call on each device looks up the device address of the scratch array (with that
//   device current).  With lazy module loading that lookup is also the moment the driver loads the
//   module, reserves the 8 MiB and takes its own locks: treat the first call per device as a
//   start-up call - make it outside of any stream capture AND outside the restricted contexts this
//   entry point is meant for (not from an allocator callback, not from a thread that must stay off
//   the allocator's lock).  `zb_norm_bwd_noalloc_init()` does only this lookup, for start-up code
//   that has nothing to compute yet.
// * All calls share the one scratch array, and the array keeps the previous call's contents
//   (every call overwrites what it later reads, so nothing needs clearing by the caller).
//   Two calls that overlap on the GPU - different streams, or different host threads - race on
//   it: serialise them.
int zb_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* stats, const void* dres,
                        void* dx, void* dw, void* db, int T, int H, int ln, int grad_f32, int accumulate,
                        cudaStream_t stream);

// Resolves (and caches) the scratch address for the current device without launching anything.
// Returns 0 on success, -2 on a CUDA error.  Call once per device at start-up.
int zb_norm_bwd_noalloc_init(void);

#ifdef __cplusplus
}
#endif
