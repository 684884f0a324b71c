// RMSNorm / LayerNorm backward, second version (same interface and scratch as zb_norm_bwd).
// Differences from the first version (norm.cu):
//   * the next row's x and dy (and its statistics) are requested before the current row is
//     reduced, and the residual gradient of the current row before its reduction, so a CTA
//     always has two rows of loads in flight instead of alternating load / reduce / store;
//   * one __syncthreads per row: the (sum g*xhat, sum g) pair is reduced in one pass, every
//     thread adds the eight warp partials itself, and the partial buffer alternates between rows;
//   * the column reduction of the per-CTA partial sums runs on H/32 CTAs of 32 x 8 threads (eight
//     rows in flight per column) instead of H/256 CTAs walking all partial rows one after another.
// Sums are formed in a fixed order, so results are deterministic.
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "norm_common.cuh"

extern "C" int zb_norm_partial_rows(int T);

namespace zb {

template <bool LN, int MAXV>
__global__ void __launch_bounds__(NORM_THREADS, MAXV <= 2 ? 2 : 1)
norm_bwd2_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                 const __nv_bfloat16* __restrict__ w, const float* __restrict__ stats,
                 const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                 float* __restrict__ part_dw, float* __restrict__ part_db, int T, int H) {
  __shared__ float2 red[2][NORM_THREADS / 32];
  const int nchunk = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float aw[MAXV][8], ab[LN ? MAXV : 1][8], wf[MAXV][8];
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) { aw[i][j] = 0.f; wf[i][j] = 0.f; }
    if (LN) {
#pragma unroll
      for (int j = 0; j < 8; ++j) ab[i][j] = 0.f;
    }
    if (c < nchunk) unpack8(wr[c], wf[i]);
  }
  uint4 cx[MAXV], cg[MAXV];
  float cmean = 0.f, crstd = 0.f;
  int row = blockIdx.x;
  if (row < T) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + size_t(row) * H);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nchunk) { cx[i] = xr[c]; cg[i] = gr[c]; }
    }
    cmean = stats[2 * row];
    crstd = stats[2 * row + 1];
  }
  int buf = 0;
  for (; row < T; row += gridDim.x, buf ^= 1) {
    // requests that do not depend on this row's reduction: next row, this row's residual gradient
    const int nrow = row + gridDim.x;
    uint4 nx[MAXV], ng[MAXV], rres[MAXV];
    float nmean = 0.f, nrstd = 0.f;
    if (nrow < T) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(nrow) * H);
      const uint4* gr = reinterpret_cast<const uint4*>(dy + size_t(nrow) * H);
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        if (c < nchunk) { nx[i] = xr[c]; ng[i] = gr[c]; }
      }
      nmean = stats[2 * nrow];
      nrstd = stats[2 * nrow + 1];
    }
    if (dres != nullptr) {
      const uint4* rr = reinterpret_cast<const uint4*>(dres + size_t(row) * H);
#pragma unroll
      for (int i = 0; i < MAXV; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        if (c < nchunk) rres[i] = rr[c];
      }
    }
    float xh[MAXV][8], g[MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nchunk) {
        float xf[8], df[8];
        unpack8(cx[i], xf);
        unpack8(cg[i], df);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xf[j] - cmean) * crstd;
          g[i][j] = df[j] * wf[i][j];
          s1 += g[i][j] * xh[i][j];
          aw[i][j] += df[j] * xh[i][j];
          if (LN) {
            s2 += g[i][j];
            ab[i][j] += df[j];
          }
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      if (LN) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane == 0) red[buf][warp] = make_float2(s1, s2);
    __syncthreads();
    float t1 = 0.f, t2 = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_THREADS / 32; ++k) {
      const float2 v = red[buf][k];
      t1 += v.x;
      t2 += v.y;
    }
    const float m1 = t1 / H, m2 = LN ? t2 / H : 0.f;
    uint4* dxr = reinterpret_cast<uint4*>(dx + size_t(row) * H);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nchunk) {
        float o[8], rf[8];
        if (dres != nullptr) unpack8(rres[i], rf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = crstd * (g[i][j] - xh[i][j] * m1 - m2);
          if (dres != nullptr) o[j] += rf[j];
        }
        dxr[c] = pack8(o);
      }
    }
#pragma unroll
    for (int i = 0; i < MAXV; ++i) { cx[i] = nx[i]; cg[i] = ng[i]; }
    cmean = nmean;
    crstd = nrstd;
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
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

// out[h] (+)= sum_p part[p, h] with a 32 x 8 thread block per 32 columns: thread (tx, ty) adds rows
// ty, ty + 8, ...; the eight partial sums of a column are then added in order by the ty = 0 thread.
template <typename OutT>
__global__ void __launch_bounds__(256)
colsum_accumulate2_kernel(const float* __restrict__ part, int P, int H, OutT* __restrict__ out, int accumulate) {
  __shared__ float sm[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int h = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (h < H) {
    for (int p = ty; p < P; p += 8) s += part[size_t(p) * H + h];
  }
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && h < H) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sm[k][tx];
    if (accumulate) t += float(out[h]);
    out[h] = OutT(t);
  }
}

}  // namespace zb

extern "C" int zb_norm_bwd2(const void* dy, const void* x, const void* w, const float* stats, const void* dres,
                            void* dx, float* part_dw, float* part_db, void* dw, void* db, int T, int H, int ln,
                            int grad_f32, int accumulate, cudaStream_t stream) {
  using namespace zb;
  if (H % 8 != 0 || H > NORM_THREADS * NORM_MAXV * 8) ZB_FAIL(-1, "norm: H=%d unsupported", H);
  if (T <= 0) return 0;
  const int P = zb_norm_partial_rows(T);
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  if (H <= NORM_THREADS * 2 * 8) {
    if (ln) norm_bwd2_kernel<true, 2><<<P, NORM_THREADS, 0, stream>>>(DY, X, W, stats, DR, DX, part_dw, part_db, T, H);
    else norm_bwd2_kernel<false, 2><<<P, NORM_THREADS, 0, stream>>>(DY, X, W, stats, DR, DX, part_dw, nullptr, T, H);
  } else {
    if (ln) norm_bwd2_kernel<true, NORM_MAXV><<<P, NORM_THREADS, 0, stream>>>(DY, X, W, stats, DR, DX, part_dw, part_db, T, H);
    else norm_bwd2_kernel<false, NORM_MAXV><<<P, NORM_THREADS, 0, stream>>>(DY, X, W, stats, DR, DX, part_dw, nullptr, T, H);
  }
  ZB_CUDA_OK(cudaGetLastError());
  const int nb = (H + 31) / 32;
  if (dw != nullptr) {
    if (grad_f32) colsum_accumulate2_kernel<float><<<nb, 256, 0, stream>>>(part_dw, P, H, static_cast<float*>(dw), accumulate);
    else colsum_accumulate2_kernel<__nv_bfloat16><<<nb, 256, 0, stream>>>(part_dw, P, H, static_cast<__nv_bfloat16*>(dw), accumulate);
  }
  if (ln && db != nullptr) {
    if (grad_f32) colsum_accumulate2_kernel<float><<<nb, 256, 0, stream>>>(part_db, P, H, static_cast<float*>(db), accumulate);
    else colsum_accumulate2_kernel<__nv_bfloat16><<<nb, 256, 0, stream>>>(part_db, P, H, static_cast<__nv_bfloat16*>(db), accumulate);
  }
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
