// RMSNorm / LayerNorm forward, second version (same interface as zb_norm_fwd): one WARP per row.
// The first version (norm.cu) gives a row to a 256-thread CTA and reduces it with three block
// barriers; here a lane keeps its share of the row (up to 32 16-byte chunks) in registers and the
// row statistics come from warp shuffles only, so a CTA of eight warps has eight independent rows
// of loads in flight and never synchronises.  Opt-in (ZORSE_NORM_FWD=2) until it has been timed.
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "norm_common.cuh"

namespace zb {

template <bool LN, int MAXC>   // MAXC 16-byte chunks per lane: H <= 32 * MAXC * 8
__global__ void __launch_bounds__(256)
norm_fwd2_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                 const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, float* __restrict__ stats,
                 int T, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const int nchunk = H >> 3;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = reinterpret_cast<const uint4*>(b);
  for (int row = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < T; row += gridDim.x * warps_per_cta) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * H);
    uint4 raw[MAXC];
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + i * 32;
      if (c < nchunk) raw[i] = xr[c];
    }
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      if (lane + i * 32 < nchunk) {
        float f[8];
        unpack8(raw[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) { s += f[j]; ss += f[j] * f[j]; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    float mean = 0.f, var;
    if (LN) {
      mean = s / H;
      float d2 = 0.f;   // two-pass variance from the registers, as the first version does
#pragma unroll
      for (int i = 0; i < MAXC; ++i) {
        if (lane + i * 32 < nchunk) {
          float f[8];
          unpack8(raw[i], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) { const float d = f[j] - mean; d2 += d * d; }
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d2 += __shfl_xor_sync(0xffffffffu, d2, o);
      var = d2 / H;
    } else {
      var = ss / H;
    }
    const float rstd = rsqrtf(var + eps);
    if (lane == 0 && stats != nullptr) {
      stats[2 * row] = mean;
      stats[2 * row + 1] = rstd;
    }
    uint4* yr = reinterpret_cast<uint4*>(y + size_t(row) * H);
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
      const int c = lane + i * 32;
      if (c < nchunk) {
        float f[8], wf[8], bf[8], o[8];
        unpack8(raw[i], f);
        unpack8(wr[c], wf);
        if (LN && b != nullptr) unpack8(br[c], bf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = (f[j] - mean) * rstd * wf[j];
          if (LN && b != nullptr) o[j] += bf[j];
        }
        yr[c] = pack8(o);
      }
    }
  }
}

}  // namespace zb

extern "C" int zb_norm_fwd2(const void* x, const void* w, const void* b, void* y, float* stats, int T, int H,
                            float eps, int ln, cudaStream_t stream) {
  using namespace zb;
  if (H % 8 != 0 || H > 32 * 32 * 8) ZB_FAIL(-1, "norm: H=%d unsupported", H);
  if (T <= 0) return 0;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto B = static_cast<const __nv_bfloat16*>(b);
  auto Y = static_cast<__nv_bfloat16*>(y);
  int blocks = (T + 7) / 8;
  const int cap = num_sms() * 8;
  if (blocks > cap) blocks = cap;
  if (H <= 32 * 16 * 8) {
    if (ln) norm_fwd2_kernel<true, 16><<<blocks, 256, 0, stream>>>(X, W, B, Y, stats, T, H, eps);
    else norm_fwd2_kernel<false, 16><<<blocks, 256, 0, stream>>>(X, W, B, Y, stats, T, H, eps);
  } else {
    if (ln) norm_fwd2_kernel<true, 32><<<blocks, 256, 0, stream>>>(X, W, B, Y, stats, T, H, eps);
    else norm_fwd2_kernel<false, 32><<<blocks, 256, 0, stream>>>(X, W, B, Y, stats, T, H, eps);
  }
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
