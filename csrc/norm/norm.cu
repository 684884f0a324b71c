// RMSNorm and LayerNorm, forward and backward, bf16 I/O with fp32 math.
// One CTA per row keeps the row in registers (16-byte loads), so every tensor is read
// once and written once.  Weight/bias gradients are reduced in two deterministic steps:
// per-CTA partial sums over a strided set of rows, then a column reduction that adds
// into the unit's gradient bucket (fp32 or bf16).
//
// Replaces the composed ATen kernels behind HF LlamaRMSNorm and nn.LayerNorm in the
// reference (models/llama_simple.py:419-422, models/gpt_simple.py:142-144).
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "norm_common.cuh"

namespace zb {

// ------------------------------- forward -------------------------------
// LN = false: y = x * rstd * w;  LN = true: y = (x - mean) * rstd * w + b.
template <bool LN>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                float* __restrict__ stats /* [T,2]: mean, rstd */, int T, int H, float eps) {
  __shared__ float red[33];
  const int row = blockIdx.x;
  const int nchunk = H >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * H);
  float v[NORM_MAXV][8];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    int c = threadIdx.x + i * NORM_THREADS;
    if (c < nchunk) {
      unpack8(xr[c], v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[i][j]; ss += v[i][j] * v[i][j]; }
    }
  }
  float mean = 0.f;
  if (LN) {
    mean = block_sum(s, red) / H;
    // two-pass variance from registers
    float d2 = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAXV; ++i) {
      int c = threadIdx.x + i * NORM_THREADS;
      if (c < nchunk) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; d2 += d * d; }
      }
    }
    ss = d2;
  }
  const float var = block_sum(ss, red) / H;
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0 && stats != nullptr) {
    stats[2 * row] = mean;
    stats[2 * row + 1] = rstd;
  }
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = reinterpret_cast<const uint4*>(b);
  uint4* yr = reinterpret_cast<uint4*>(y + size_t(row) * H);
#pragma unroll
  for (int i = 0; i < NORM_MAXV; ++i) {
    int c = threadIdx.x + i * NORM_THREADS;
    if (c < nchunk) {
      float wf[8], bf[8], o[8];
      unpack8(wr[c], wf);
      if (LN && b != nullptr) unpack8(br[c], bf);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = (v[i][j] - mean) * rstd * wf[j];
        if (LN && b != nullptr) o[j] += bf[j];
      }
      yr[c] = pack8(o);
    }
  }
}

// ------------------------------- backward -------------------------------
// dx = (dres) + rstd * (g - xhat * mean(g * xhat) [- mean(g)]) with g = dy * w.
// Each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and keeps its partial
// dw (and db) in registers; partials go to part_dw[gridDim.x, H] (and part_db).
template <bool LN, int MAXV>
__global__ void __launch_bounds__(NORM_THREADS, MAXV <= 2 ? 2 : 1)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ stats,
                const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                float* __restrict__ part_dw, float* __restrict__ part_db, int T, int H) {
  __shared__ float red[33];
  const int nchunk = H >> 3;
  float aw[MAXV][8], ab[MAXV][8], wf[MAXV][8];
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int c = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) { aw[i][j] = 0.f; ab[i][j] = 0.f; wf[i][j] = 0.f; }
    if (c < nchunk) unpack8(wr[c], wf[i]);
  }
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + size_t(row) * H);
    const float mean = stats[2 * row], rstd = stats[2 * row + 1];
    float xh[MAXV][8], g[MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int c = threadIdx.x + i * NORM_THREADS;
      if (c < nchunk) {
        float xf[8], df[8];
        unpack8(xr[c], xf);
        unpack8(gr[c], df);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xf[j] - mean) * rstd;
          g[i][j] = df[j] * wf[i][j];
          s1 += g[i][j] * xh[i][j];
          s2 += g[i][j];
          aw[i][j] += df[j] * xh[i][j];
          ab[i][j] += df[j];
        }
      }
    }
    const float m1 = block_sum(s1, red) / H;
    float m2 = 0.f;
    if (LN) m2 = block_sum(s2, red) / H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + size_t(row) * H);
    const uint4* rr = reinterpret_cast<const uint4*>(dres ? dres + size_t(row) * H : nullptr);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int c = threadIdx.x + i * NORM_THREADS;
      if (c < nchunk) {
        float o[8], rf[8];
        if (dres) unpack8(rr[c], rf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = rstd * (g[i][j] - xh[i][j] * m1 - m2);
          if (dres) o[j] += rf[j];
        }
        dxr[c] = pack8(o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int c = threadIdx.x + i * NORM_THREADS;
    if (c < nchunk) {
      float4* pw = reinterpret_cast<float4*>(part_dw + size_t(blockIdx.x) * H + c * 8);
      pw[0] = make_float4(aw[i][0], aw[i][1], aw[i][2], aw[i][3]);
      pw[1] = make_float4(aw[i][4], aw[i][5], aw[i][6], aw[i][7]);
      if (LN && part_db != nullptr) {
        float4* pb = reinterpret_cast<float4*>(part_db + size_t(blockIdx.x) * H + c * 8);
        pb[0] = make_float4(ab[i][0], ab[i][1], ab[i][2], ab[i][3]);
        pb[1] = make_float4(ab[i][4], ab[i][5], ab[i][6], ab[i][7]);
      }
    }
  }
}

// out[h] (+)= sum_p part[p, h]; out is fp32 or bf16.
template <typename OutT>
__global__ void colsum_accumulate_kernel(const float* __restrict__ part, int P, int H,
                                         OutT* __restrict__ out, int accumulate) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += part[size_t(p) * H + h];
  if (accumulate) s += float(out[h]);
  out[h] = OutT(s);
}

// Column sums of a bf16 matrix [T, N] (bias gradients): partial sums per CTA over a
// strided set of rows, finished by colsum_accumulate_kernel.
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ dy, int T, int N, int ld,
                      float* __restrict__ part) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= N) return;
  float s = 0.f;
  for (int r = blockIdx.y; r < T; r += gridDim.y) s += __bfloat162float(dy[size_t(r) * ld + col]);
  part[size_t(blockIdx.y) * N + col] = s;
}

}  // namespace zb

namespace zb {
int norm_bwd_with_scratch(const void* dy, const void* x, const void* w, const float* stats, const void* dres, void* dx,
                          float* part_dw, float* part_db, int P, void* dw, void* db, int T, int H, int ln, int grad_f32,
                          int accumulate, cudaStream_t stream);
}  // namespace zb

extern "C" {

int zb_norm_partial_rows(int T) {
  int n = zb::num_sms() * 2;
  return T < n ? T : n;
}

// stats: fp32 [T, 2]; ln: 0 = RMSNorm (bias ignored), 1 = LayerNorm.
int zb_norm_fwd(const void* x, const void* w, const void* b, void* y, float* stats, int T, int H,
                float eps, int ln, cudaStream_t stream) {
  using namespace zb;
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAXV * 8) ZB_FAIL(-1, "norm: H=%d unsupported", H);
  if (T <= 0) return 0;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto B = static_cast<const __nv_bfloat16*>(b);
  auto Y = static_cast<__nv_bfloat16*>(y);
  if (ln) norm_fwd_kernel<true><<<T, NORM_THREADS, 0, stream>>>(X, W, B, Y, stats, T, H, eps);
  else norm_fwd_kernel<false><<<T, NORM_THREADS, 0, stream>>>(X, W, B, Y, stats, T, H, eps);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

// part_dw / part_db: fp32 scratch [zb_norm_partial_rows(T), H]. dw/db: gradient slots
// (fp32 if grad_f32 else bf16) that are accumulated into when `accumulate` is set.
int zb_norm_bwd(const void* dy, const void* x, const void* w, const float* stats, const void* dres,
                void* dx, float* part_dw, float* part_db, void* dw, void* db, int T, int H, int ln,
                int grad_f32, int accumulate, cudaStream_t stream) {
  using namespace zb;
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAXV * 8) ZB_FAIL(-1, "norm: H=%d unsupported", H);
  if (T <= 0) return 0;
  return norm_bwd_with_scratch(dy, x, w, stats, dres, dx, part_dw, part_db, zb_norm_partial_rows(T), dw, db, T, H, ln,
                               grad_f32, accumulate, stream);
}

// Bias gradient: out[n] (+)= sum_t dy[t, n]. part: fp32 scratch [64, N].
int zb_colsum(const void* dy, int T, int N, int ld, float* part, void* out, int grad_f32,
              int accumulate, cudaStream_t stream) {
  using namespace zb;
  if (T <= 0 || N <= 0) return 0;
  const int P = T < 64 ? T : 64;
  dim3 grid((N + 255) / 256, P);
  colsum_partial_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dy), T, N, ld, part);
  const int nb = (N + 255) / 256;
  if (grad_f32) colsum_accumulate_kernel<float><<<nb, 256, 0, stream>>>(part, P, N, static_cast<float*>(out), accumulate);
  else colsum_accumulate_kernel<__nv_bfloat16><<<nb, 256, 0, stream>>>(part, P, N, static_cast<__nv_bfloat16*>(out), accumulate);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"

// Launch sequence of the norm backward with caller-provided scratch and partial-row count
// (used by the allocation-free entry point in norm_bwd_noalloc.cu).
namespace zb {
int norm_bwd_with_scratch(const void* dy, const void* x, const void* w, const float* stats, const void* dres, void* dx,
                          float* part_dw, float* part_db, int P, void* dw, void* db, int T, int H, int ln, int grad_f32,
                          int accumulate, cudaStream_t stream) {
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  // rows up to 4096 wide need two 16-byte chunks per thread: half the registers, two CTAs per SM
  if (H <= NORM_THREADS * 2 * 8) {
    if (ln) norm_bwd_kernel<true, 2><<<P, NORM_THREADS, 0, stream>>>(DY, X, W, stats, DR, DX, part_dw, part_db, T, H);
    else norm_bwd_kernel<false, 2><<<P, NORM_THREADS, 0, stream>>>(DY, X, W, stats, DR, DX, part_dw, nullptr, T, H);
  } else {
    if (ln) norm_bwd_kernel<true, NORM_MAXV><<<P, NORM_THREADS, 0, stream>>>(DY, X, W, stats, DR, DX, part_dw, part_db, T, H);
    else norm_bwd_kernel<false, NORM_MAXV><<<P, NORM_THREADS, 0, stream>>>(DY, X, W, stats, DR, DX, part_dw, nullptr, T, H);
  }
  ZB_CUDA_OK(cudaGetLastError());
  const int nb = (H + 255) / 256;
  if (dw != nullptr) {
    if (grad_f32) colsum_accumulate_kernel<float><<<nb, 256, 0, stream>>>(part_dw, P, H, static_cast<float*>(dw), accumulate);
    else colsum_accumulate_kernel<__nv_bfloat16><<<nb, 256, 0, stream>>>(part_dw, P, H, static_cast<__nv_bfloat16*>(dw), accumulate);
  }
  if (ln && db != nullptr) {
    if (grad_f32) colsum_accumulate_kernel<float><<<nb, 256, 0, stream>>>(part_db, P, H, static_cast<float*>(db), accumulate);
    else colsum_accumulate_kernel<__nv_bfloat16><<<nb, 256, 0, stream>>>(part_db, P, H, static_cast<__nv_bfloat16*>(db), accumulate);
  }
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
}  // namespace zb
