// Fused Adam on a flat fp32 shard: one pass reads p, m, v, g and writes p, m, v plus the
// refreshed bf16 copy of the parameters that the next all-gather sends.  Gradients may be
// fp32 or bf16 and are scaled by grad_scale first; with zero_grad the gradient slot is
// cleared in the same pass.  Arithmetic follows torch.optim.Adam (the reference builds
// torch.optim.Adam(fused=True), zorse.py:88-90, zorse_utils/pipeline.py:176-179).
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2_sqrt, grad_scale;
};

__device__ __forceinline__ float adam_update(float& p, float& m, float& v, float g, const AdamHyper& h) {
  g *= h.grad_scale;
  if (h.weight_decay != 0.f) g += h.weight_decay * p;
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  const float denom = sqrtf(v) / h.bc2_sqrt + h.eps;
  p -= (h.lr / h.bc1) * (m / denom);
  return p;
}

template <typename GT>
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, GT* __restrict__ g,
            __nv_bfloat16* __restrict__ p16, long n, AdamHyper h, int zero_grad) {
  const long n4 = n >> 2;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n4; i += long(gridDim.x) * blockDim.x) {
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float gg[4];
    if (sizeof(GT) == 4) {
      float4 t = reinterpret_cast<const float4*>(g)[i];
      gg[0] = t.x; gg[1] = t.y; gg[2] = t.z; gg[3] = t.w;
      if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      uint2 t = reinterpret_cast<const uint2*>(g)[i];
      float2 a = unpack_bf16x2(t.x), b = unpack_bf16x2(t.y);
      gg[0] = a.x; gg[1] = a.y; gg[2] = b.x; gg[3] = b.y;
      if (zero_grad) reinterpret_cast<uint2*>(g)[i] = make_uint2(0u, 0u);
    }
    adam_update(pp.x, mm.x, vv.x, gg[0], h);
    adam_update(pp.y, mm.y, vv.y, gg[1], h);
    adam_update(pp.z, mm.z, vv.z, gg[2], h);
    adam_update(pp.w, mm.w, vv.w, gg[3], h);
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (p16 != nullptr)
      reinterpret_cast<uint2*>(p16)[i] = make_uint2(pack_bf16x2(pp.x, pp.y), pack_bf16x2(pp.z, pp.w));
  }
  // tail (n not a multiple of 4)
  const long tail0 = n4 << 2;
  for (long i = tail0 + blockIdx.x * long(blockDim.x) + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) {
    float pp = p[i], mm = m[i], vv = v[i];
    float gg = float(g[i]);
    if (zero_grad) g[i] = GT(0.f);
    adam_update(pp, mm, vv, gg, h);
    p[i] = pp; m[i] = mm; v[i] = vv;
    if (p16 != nullptr) p16[i] = __float2bfloat16(pp);
  }
}

}  // namespace zb

extern "C" int zb_adam(float* p, float* m, float* v, void* g, void* p16, long n, float lr, float beta1,
                       float beta2, float eps, float weight_decay, int step, float grad_scale, int grad_f32,
                       int zero_grad, cudaStream_t stream) {
  using namespace zb;
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(g)) & 15)
    ZB_FAIL(-1, "adam: buffers must be 16-byte aligned");
  if (p16 && (reinterpret_cast<uintptr_t>(p16) & 7)) ZB_FAIL(-1, "adam: bf16 copy must be 8-byte aligned");
  AdamHyper h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.weight_decay = weight_decay;
  h.bc1 = 1.f - powf(beta1, float(step));
  h.bc2_sqrt = sqrtf(1.f - powf(beta2, float(step)));
  h.grad_scale = grad_scale;
  long blocks = (n / 4 + 255) / 256;
  long cap = long(num_sms()) * 8;
  int grid = int(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  if (grad_f32)
    adam_kernel<float><<<grid, 256, 0, stream>>>(p, m, v, static_cast<float*>(g), static_cast<__nv_bfloat16*>(p16),
                                                 n, h, zero_grad);
  else
    adam_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p, m, v, static_cast<__nv_bfloat16*>(g),
                                                         static_cast<__nv_bfloat16*>(p16), n, h, zero_grad);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
