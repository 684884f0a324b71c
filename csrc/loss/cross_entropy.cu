// Fused cross-entropy forward + backward over bf16 logits [T, V]:
//   loss[t]    = logsumexp(logits[t, :]) - logits[t, target[t]]
//   dlogits    = (softmax(logits[t, :]) - onehot(target[t])) * grad_scale      (bf16)
// One CTA per row; the row is read twice (the second read hits L2) and the gradient is
// written once, in place if dlogits == logits.  Replaces F.cross_entropy + its autograd
// (reference call site zorse_utils/pipeline_schedule_v2.py:182-184).
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ void ce_unpack8(const uint4& u, float* f) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const long* __restrict__ targets,
                  __nv_bfloat16* __restrict__ dlogits, float* __restrict__ loss_rows, int T, int V,
                  long ld, float grad_scale, long ignore_index) {
  __shared__ float red_m[CE_THREADS / 32], red_s[CE_THREADS / 32];
  __shared__ float bc[2];
  const int row = blockIdx.x;
  const __nv_bfloat16* x = logits + row * ld;
  const bool vec = (V % 8 == 0) && (ld % 8 == 0);
  float m = -INFINITY, s = 0.f;
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int c = threadIdx.x; c < V / 8; c += CE_THREADS) {
      float f[8];
      ce_unpack8(xv[c], f);
      float cm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
      if (cm > m) { s *= __expf(m - cm); m = cm; }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
    }
  } else {
    for (int c = threadIdx.x; c < V; c += CE_THREADS) {
      float f = __bfloat162float(x[c]);
      if (f > m) { s *= __expf(m - f); m = f; }
      s += __expf(f - m);
    }
  }
  // combine (m, s) across the CTA
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) { red_m[threadIdx.x >> 5] = m; red_s[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < CE_THREADS / 32 ? red_m[threadIdx.x] : -INFINITY;
    s = threadIdx.x < CE_THREADS / 32 ? red_s[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      float nm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
      m = nm;
    }
    if (threadIdx.x == 0) { bc[0] = m; bc[1] = s; }
  }
  __syncthreads();
  m = bc[0];
  s = bc[1];
  const long tgt = targets[row];
  const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
  if (threadIdx.x == 0) {
    float l = 0.f;
    if (!ignored) l = (m + __logf(s)) - __bfloat162float(x[tgt]);
    loss_rows[row] = l;
  }
  if (dlogits == nullptr) return;
  const float inv = ignored ? 0.f : grad_scale / s;
  const float gs = ignored ? 0.f : grad_scale;
  __nv_bfloat16* dx = dlogits + row * ld;
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    uint4* dv = reinterpret_cast<uint4*>(dx);
    for (int c = threadIdx.x; c < V / 8; c += CE_THREADS) {
      float f[8];
      ce_unpack8(xv[c], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = __expf(f[j] - m) * inv;
        if (c * 8 + j == tgt) f[j] -= gs;
      }
      uint4 o;
      o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
      o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
      dv[c] = o;
    }
  } else {
    for (int c = threadIdx.x; c < V; c += CE_THREADS) {
      float f = __expf(__bfloat162float(x[c]) - m) * inv;
      if (c == tgt) f -= gs;
      dx[c] = __float2bfloat16(f);
    }
  }
}

}  // namespace zb

extern "C" int zb_cross_entropy(const void* logits, const long* targets, void* dlogits, float* loss_rows,
                                int T, int V, long ld, float grad_scale, long ignore_index,
                                cudaStream_t stream) {
  using namespace zb;
  if (T <= 0) return 0;
  ce_fwd_bwd_kernel<<<T, CE_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), targets,
                                                  static_cast<__nv_bfloat16*>(dlogits), loss_rows, T, V, ld,
                                                  grad_scale, ignore_index);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
