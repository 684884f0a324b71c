// Memory-bound elementwise kernels (bf16 I/O, fp32 math, 16-byte accesses):
//   RoPE (rotate-half, in place on the packed QKV buffer), SwiGLU fwd/bwd,
//   GELU(tanh)/ReLU fwd/bwd, embedding gather / scatter-add (+ learned positions).
// They stand in for the ATen elementwise kernels the reference reaches through
// apply_rotary_pos_emb (models/llama_simple.py:34-58), HF LlamaMLP, gelu_new
// (models/gpt_simple.py:119-134) and nn.Embedding (models/llama_simple.py:550-552).
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

__device__ __forceinline__ void unpack8e(const uint4& u, float* f) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8e(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// ------------------------------- RoPE -------------------------------
// buf: [T, row_stride] bf16; heads 0..nheads-1 of width d start at column 0 (q heads then
// k heads in the packed QKV layout). cs: [S, d] fp32 = cos(d/2) | sin(d/2) per position.
// position of token t = (t % S). sign = +1 forward, -1 backward (transpose rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ buf, const float* __restrict__ cs, int T,
                            int S, int nheads, int d, int row_stride, float sign) {
  const int half = d >> 1;
  const int cpr = half >> 3;  // 16-byte chunks per half head
  const long total = long(T) * nheads * cpr;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int c = int(i % cpr);
    const int h = int((i / cpr) % nheads);
    const int t = int(i / (long(cpr) * nheads));
    const int pos = t % S;
    __nv_bfloat16* base = buf + size_t(t) * row_stride + h * d + c * 8;
    uint4 lo = *reinterpret_cast<uint4*>(base);
    uint4 hi = *reinterpret_cast<uint4*>(base + half);
    float a[8], b[8], oa[8], ob[8];
    unpack8e(lo, a);
    unpack8e(hi, b);
    const float4* cp = reinterpret_cast<const float4*>(cs + size_t(pos) * d + c * 8);
    const float4* sp = reinterpret_cast<const float4*>(cs + size_t(pos) * d + half + c * 8);
    float co[8], si[8];
    *reinterpret_cast<float4*>(co) = cp[0]; *reinterpret_cast<float4*>(co + 4) = cp[1];
    *reinterpret_cast<float4*>(si) = sp[0]; *reinterpret_cast<float4*>(si + 4) = sp[1];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float s = si[j] * sign;
      oa[j] = a[j] * co[j] - b[j] * s;
      ob[j] = b[j] * co[j] + a[j] * s;
    }
    *reinterpret_cast<uint4*>(base) = pack8e(oa);
    *reinterpret_cast<uint4*>(base + half) = pack8e(ob);
  }
}

// ------------------------------- SwiGLU -------------------------------
// gu: [T, 2F] (gate | up), out: [T, F] = silu(gate) * up
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                  long T, int F) {
  const int cpr = F >> 3;
  const long total = T * cpr;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const long t = i / cpr;
    const int c = int(i % cpr);
    const __nv_bfloat16* g = gu + t * 2 * F + c * 8;
    float a[8], b[8], o[8];
    unpack8e(ld_nc_v4(g), a);
    unpack8e(ld_nc_v4(g + F), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = a[j] / (1.f + __expf(-a[j])) * b[j];
    *reinterpret_cast<uint4*>(out + t * F + c * 8) = pack8e(o);
  }
}
// dgu: [T, 2F]: dgate = dout * up * silu'(gate), dup = dout * silu(gate)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long T, int F) {
  const int cpr = F >> 3;
  const long total = T * cpr;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const long t = i / cpr;
    const int c = int(i % cpr);
    const __nv_bfloat16* g = gu + t * 2 * F + c * 8;
    float a[8], b[8], d[8], da[8], db[8];
    unpack8e(ld_nc_v4(g), a);
    unpack8e(ld_nc_v4(g + F), b);
    unpack8e(ld_nc_v4(dout + t * F + c * 8), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float sg = 1.f / (1.f + __expf(-a[j]));
      float silu = a[j] * sg;
      da[j] = d[j] * b[j] * (sg * (1.f + a[j] * (1.f - sg)));
      db[j] = d[j] * silu;
    }
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + c * 8) = pack8e(da);
    *reinterpret_cast<uint4*>(dgu + t * 2 * F + F + c * 8) = pack8e(db);
  }
}

// ------------------------------- GELU / ReLU -------------------------------
// kind: 0 = tanh GELU ("gelu_new"), 1 = ReLU, 2 = erf GELU
__device__ __forceinline__ float act_fwd(float x, int kind) {
  if (kind == 1) return fmaxf(x, 0.f);
  if (kind == 2) return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float act_bwd(float x, int kind) {
  if (kind == 1) return x > 0.f ? 1.f : 0.f;
  if (kind == 2) {
    float cdf = 0.5f * (1.f + erff(x * 0.7071067811865476f));
    return cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  float th = tanhf(u);
  return 0.5f * (1.f + th) + 0.5f * x * (1.f - th * th) * k0 * (1.f + 3.f * k1 * x * x);
}
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long n8, int kind) {
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n8; i += long(gridDim.x) * blockDim.x) {
    float a[8], o[8];
    unpack8e(ld_nc_v4(x + i * 8), a);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_fwd(a[j], kind);
    *reinterpret_cast<uint4*>(y + i * 8) = pack8e(o);
  }
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                               __nv_bfloat16* __restrict__ dx, long n8, int kind) {
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < n8; i += long(gridDim.x) * blockDim.x) {
    float a[8], d[8], o[8];
    unpack8e(ld_nc_v4(x + i * 8), a);
    unpack8e(ld_nc_v4(dy + i * 8), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = d[j] * act_bwd(a[j], kind);
    *reinterpret_cast<uint4*>(dx + i * 8) = pack8e(o);
  }
}

// ------------------------------- embedding -------------------------------
// out[t, :] = table[ids[t], :] (+ pos_table[(t % S) + pos_offset, :])
__global__ void embedding_fwd_kernel(const long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     const __nv_bfloat16* __restrict__ pos_table, __nv_bfloat16* __restrict__ out,
                                     int T, int H, int V, int S, int pos_offset) {
  const int cpr = H >> 3;
  const long total = long(T) * cpr;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int t = int(i / cpr), c = int(i % cpr);
    long id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    uint4 v = *reinterpret_cast<const uint4*>(table + id * H + c * 8);
    if (pos_table != nullptr) {
      float a[8], b[8];
      unpack8e(v, a);
      unpack8e(*reinterpret_cast<const uint4*>(pos_table + size_t((t % S) + pos_offset) * H + c * 8), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += b[j];
      v = pack8e(a);
    }
    *reinterpret_cast<uint4*>(out + size_t(t) * H + c * 8) = v;
  }
}
// dtable[ids[t], :] += dout[t, :] (atomic), dpos[(t % S) + off, :] += dout[t, :]
template <typename GT>
__device__ __forceinline__ void atomic_add2(GT* p, float a, float b);
template <>
__device__ __forceinline__ void atomic_add2<float>(float* p, float a, float b) {
  atomicAdd(p, a);
  atomicAdd(p + 1, b);
}
template <>
__device__ __forceinline__ void atomic_add2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  atomicAdd(reinterpret_cast<__nv_bfloat162*>(p), __floats2bfloat162_rn(a, b));
}
template <typename GT>
__global__ void embedding_bwd_kernel(const long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     GT* __restrict__ dtable, GT* __restrict__ dpos, int T, int H, int V,
                                     int S, int pos_offset) {
  const int cpr = H >> 3;
  const long total = long(T) * cpr;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const int t = int(i / cpr), c = int(i % cpr);
    long id = ids[t];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    float a[8];
    unpack8e(ld_nc_v4(dout + size_t(t) * H + c * 8), a);
    GT* dst = dtable + id * H + c * 8;
#pragma unroll
    for (int j = 0; j < 8; j += 2) atomic_add2<GT>(dst + j, a[j], a[j + 1]);
    if (dpos != nullptr) {
      GT* dp = dpos + size_t((t % S) + pos_offset) * H + c * 8;
#pragma unroll
      for (int j = 0; j < 8; j += 2) atomic_add2<GT>(dp + j, a[j], a[j + 1]);
    }
  }
}

static inline int grid_for(long work_items, int threads) {
  long b = (work_items + threads - 1) / threads;
  long cap = long(num_sms()) * 16;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace zb

extern "C" {

int zb_rope(void* buf, const float* cs, int T, int S, int nheads, int d, int row_stride, int backward,
            cudaStream_t stream) {
  using namespace zb;
  if (d % 16 != 0 || row_stride % 8 != 0) ZB_FAIL(-1, "rope: head dim %d / stride %d unsupported", d, row_stride);
  if (T <= 0 || nheads <= 0) return 0;
  long total = long(T) * nheads * (d / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(buf), cs, T, S, nheads, d,
                                                       row_stride, backward ? -1.f : 1.f);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

int zb_swiglu_fwd(const void* gu, void* out, long T, int F, cudaStream_t stream) {
  using namespace zb;
  if (F % 8 != 0) ZB_FAIL(-1, "swiglu: F=%d not a multiple of 8", F);
  if (T <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), T, F);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
int zb_swiglu_bwd(const void* gu, const void* dout, void* dgu, long T, int F, cudaStream_t stream) {
  using namespace zb;
  if (F % 8 != 0) ZB_FAIL(-1, "swiglu: F=%d not a multiple of 8", F);
  if (T <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dout),
      static_cast<__nv_bfloat16*>(dgu), T, F);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
int zb_act_fwd(const void* x, void* y, long n, int kind, cudaStream_t stream) {
  using namespace zb;
  if (n % 8 != 0) ZB_FAIL(-1, "act: n=%ld not a multiple of 8", n);
  if (n <= 0) return 0;
  act_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                          static_cast<__nv_bfloat16*>(y), n / 8, kind);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
int zb_act_bwd(const void* x, const void* dy, void* dx, long n, int kind, cudaStream_t stream) {
  using namespace zb;
  if (n % 8 != 0) ZB_FAIL(-1, "act: n=%ld not a multiple of 8", n);
  if (n <= 0) return 0;
  act_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                          static_cast<const __nv_bfloat16*>(dy),
                                                          static_cast<__nv_bfloat16*>(dx), n / 8, kind);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
int zb_embedding_fwd(const long* ids, const void* table, const void* pos_table, void* out, int T, int H, int V,
                     int S, int pos_offset, cudaStream_t stream) {
  using namespace zb;
  if (H % 8 != 0) ZB_FAIL(-1, "embedding: H=%d not a multiple of 8", H);
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<grid_for(long(T) * (H / 8), 256), 256, 0, stream>>>(
      ids, static_cast<const __nv_bfloat16*>(table), static_cast<const __nv_bfloat16*>(pos_table),
      static_cast<__nv_bfloat16*>(out), T, H, V, S, pos_offset);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
int zb_embedding_bwd(const long* ids, const void* dout, void* dtable, void* dpos, int T, int H, int V, int S,
                     int pos_offset, int grad_f32, cudaStream_t stream) {
  using namespace zb;
  if (H % 8 != 0) ZB_FAIL(-1, "embedding: H=%d not a multiple of 8", H);
  if (T <= 0) return 0;
  const int g = grid_for(long(T) * (H / 8), 256);
  if (grad_f32)
    embedding_bwd_kernel<float><<<g, 256, 0, stream>>>(ids, static_cast<const __nv_bfloat16*>(dout),
                                                       static_cast<float*>(dtable), static_cast<float*>(dpos), T,
                                                       H, V, S, pos_offset);
  else
    embedding_bwd_kernel<__nv_bfloat16><<<g, 256, 0, stream>>>(
        ids, static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dtable),
        static_cast<__nv_bfloat16*>(dpos), T, H, V, S, pos_offset);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
