// Fused reduce-scatter + cast/scale + sharded Adam over NVLink peer memory.
//
// Every rank of a shard group keeps the unit's full gradient bucket (bf16 or fp32) in
// symmetric memory, so each rank can address its peers' buckets directly.  Rank r owns
// elements [r*n/R, (r+1)*n/R): this kernel loads that slice from all R buckets with plain
// 16-byte peer loads (fixed rank order -> deterministic sum), scales it, runs Adam on the
// fp32 master / m / v shard and writes the refreshed bf16 parameter shard the next
// all-gather sends.  One pass: no reduced-gradient tensor, no separate cast, no separate
// optimizer launch.  (Reference: dist.reduce_scatter_tensor + cast + fused Adam,
// utils/patch.py:585-589, 99-143.)
//
// Cross-GPU ordering uses three int flags per (unit, rank) in symmetric memory, written
// with st.release.sys by the producer and polled with ld.acquire.sys by the consumer:
//   ready[p]   rank p finished accumulating the unit's gradients for epoch e
//   done[p]    rank p finished reading its slice of everybody's bucket for epoch e
//   version[p] rank p's bf16 shard holds the parameters of epoch e
// Every wait is bounded; on a timeout the kernel records ST_TIMEOUT_FLAG and returns
// without touching the optimizer state.
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

constexpr int MAX_R = 8;

struct RsAdamParams {
  const void* grad[MAX_R];  // bucket base of every rank of the group (own one included)
  const void* grad_mc;      // NVLS variants: the buckets' multicast address (one load returns the sum over all ranks)
  __nv_bfloat16* p16_mc;    // push variant: multicast address of this rank's shard inside the unsharded buffers
  int* flags[MAX_R];        // flag block of every rank: [3][R] ints (ready, done, version)
  int R, r;
  long shard_n;             // elements per shard
  float* master; float* m; float* v;
  __nv_bfloat16* p16;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2_sqrt, grad_scale;
  int epoch;
  int* status;
  unsigned int* counter;    // zeroed int in local memory (last-block detection)
  unsigned long long wait_ns;
};

template <typename GT> struct GradVec;
template <> struct GradVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ void load(const float* p, float* f) { unpack(ld_v4_relaxed_sys(p), f); }
};
template <> struct GradVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) { unpack(ld_v4_relaxed_sys(p), f); }
};

// In-switch reduction: one multimem.ld_reduce on the multicast address of the buckets returns the
// sum over all ranks of the group (NVSwitch adds the R copies; bf16 inputs are accumulated in fp32
// and returned as bf16), so 1/R of the bytes of the peer-load variants arrive at this GPU.
template <typename GT> struct NvlsVec;
template <> struct NvlsVec<float> {
  static __device__ __forceinline__ uint4 load(const void* mc) {
    uint4 u;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(mc) : "memory");
    return u;
  }
};
template <> struct NvlsVec<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 load(const void* mc) {
    uint4 u;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(mc) : "memory");
    return u;
  }
};

__device__ __forceinline__ void multimem_st_v4(void* mc, const uint4& u) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(u.x), "r"(u.y), "r"(u.z),
               "r"(u.w)
               : "memory");
}
__device__ __forceinline__ void multimem_st_v2(void* mc, const uint2& u) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc), "r"(u.x), "r"(u.y) : "memory");
}

enum : int { RS_PLAIN = 0, RS_EARLY = 1, RS_NVLS = 2, RS_NVLS_PUSH = 3 };

// MODE = RS_PLAIN: the measured kernel (peer loads one after another, then the optimizer state).
// MODE = RS_EARLY (candidate, selected with zb_set_rs_adam_variant(1)): the optimizer state and all
// R slices are requested before anything is consumed, so one NVLink round trip covers them all.
// MODE = RS_NVLS (candidate, zb_rs_adam_nvls): the slice is reduced inside NVSwitch.
// MODE = RS_NVLS_PUSH (candidate, zb_rs_adam_nvls with p16_mc): as RS_NVLS, and the refreshed bf16
// shard is stored through the multicast address of the unsharded parameter buffers, so it lands in
// every rank's copy (this rank's included) and the next step needs no all-gather: reduce-scatter,
// optimizer and all-gather are this one kernel.  Safe because a rank announces `ready` only after
// its last use of the unit's parameters in the step; `version` tells the peers that the shard arrived.
template <typename GT, int MODE>
__global__ void __launch_bounds__(256)
rs_adam_kernel(const RsAdamParams p) {
  constexpr int N = GradVec<GT>::N;
  constexpr bool EARLY = MODE == RS_EARLY;
  __shared__ int s_ok;
  // 1. announce that this rank's bucket is complete (the launch is stream-ordered after the
  //    last wgrad kernel of the unit), then wait for everybody else's announcement.
  if (blockIdx.x == 0 && threadIdx.x < p.R) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + 0 * p.R + p.r, p.epoch);
  }
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int q = 0; q < p.R && ok; ++q)
      ok = flag_wait_ge(p.flags[p.r] + 0 * p.R + q, p.epoch, p.wait_ns, p.status, ST_TIMEOUT_FLAG);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  // A block whose wait ran out (the status word says so) skips the arithmetic but still takes part
  // in the block count below, so that the counter is back at zero for the unit's next launch.
  const long nvec = s_ok ? p.shard_n / N : 0;

  // 2. reduce + Adam over this rank's slice
  const long lo = long(p.r) * p.shard_n;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < nvec; i += long(gridDim.x) * blockDim.x) {
    if (!zb_in_bounds(lo + (i + 1) * N <= long(p.R) * p.shard_n && p.r >= 0 && p.r < p.R, p.status, 5)) break;
    float g[N];
    float pm[N], mm[N], vv[N];
#pragma unroll
    for (int k = 0; k < N; ++k) g[k] = 0.f;
    if (MODE == RS_NVLS || MODE == RS_NVLS_PUSH) {
#pragma unroll
      for (int k = 0; k < N; k += 4) {
        *reinterpret_cast<float4*>(pm + k) = *reinterpret_cast<const float4*>(p.master + i * N + k);
        *reinterpret_cast<float4*>(mm + k) = *reinterpret_cast<const float4*>(p.m + i * N + k);
        *reinterpret_cast<float4*>(vv + k) = *reinterpret_cast<const float4*>(p.v + i * N + k);
      }
      GradVec<GT>::unpack(NvlsVec<GT>::load(static_cast<const GT*>(p.grad_mc) + lo + i * N), g);
    } else if (EARLY) {
#pragma unroll
      for (int k = 0; k < N; k += 4) {
        *reinterpret_cast<float4*>(pm + k) = *reinterpret_cast<const float4*>(p.master + i * N + k);
        *reinterpret_cast<float4*>(mm + k) = *reinterpret_cast<const float4*>(p.m + i * N + k);
        *reinterpret_cast<float4*>(vv + k) = *reinterpret_cast<const float4*>(p.v + i * N + k);
      }
      uint4 raw[MAX_R];
#pragma unroll
      for (int q = 0; q < MAX_R; ++q)
        if (q < p.R) raw[q] = ld_v4_relaxed_sys(static_cast<const GT*>(p.grad[q]) + lo + i * N);
#pragma unroll
      for (int q = 0; q < MAX_R; ++q) {     // same rank order as the other variant: same sum
        if (q < p.R) {
          float t[N];
          GradVec<GT>::unpack(raw[q], t);
#pragma unroll
          for (int k = 0; k < N; ++k) g[k] += t[k];
        }
      }
    } else {
      for (int q = 0; q < p.R; ++q) {
        float t[N];
        GradVec<GT>::load(static_cast<const GT*>(p.grad[q]) + lo + i * N, t);
#pragma unroll
        for (int k = 0; k < N; ++k) g[k] += t[k];
      }
#pragma unroll
      for (int k = 0; k < N; k += 4) {
        *reinterpret_cast<float4*>(pm + k) = *reinterpret_cast<const float4*>(p.master + i * N + k);
        *reinterpret_cast<float4*>(mm + k) = *reinterpret_cast<const float4*>(p.m + i * N + k);
        *reinterpret_cast<float4*>(vv + k) = *reinterpret_cast<const float4*>(p.v + i * N + k);
      }
    }
#pragma unroll
    for (int k = 0; k < N; ++k) {
      float gg = g[k] * p.grad_scale;
      if (p.weight_decay != 0.f) gg += p.weight_decay * pm[k];
      mm[k] = p.beta1 * mm[k] + (1.f - p.beta1) * gg;
      vv[k] = p.beta2 * vv[k] + (1.f - p.beta2) * gg * gg;
      pm[k] -= (p.lr / p.bc1) * (mm[k] / (sqrtf(vv[k]) / p.bc2_sqrt + p.eps));
    }
#pragma unroll
    for (int k = 0; k < N; k += 4) {
      *reinterpret_cast<float4*>(p.master + i * N + k) = *reinterpret_cast<float4*>(pm + k);
      *reinterpret_cast<float4*>(p.m + i * N + k) = *reinterpret_cast<float4*>(mm + k);
      *reinterpret_cast<float4*>(p.v + i * N + k) = *reinterpret_cast<float4*>(vv + k);
    }
    if (N == 8) {
      uint4 u;
      u.x = pack_bf16x2(pm[0], pm[1]); u.y = pack_bf16x2(pm[2], pm[3]);
      u.z = pack_bf16x2(pm[4], pm[5]); u.w = pack_bf16x2(pm[6], pm[7]);
      if (MODE == RS_NVLS_PUSH) multimem_st_v4(p.p16_mc + i * N, u);
      else *reinterpret_cast<uint4*>(p.p16 + i * N) = u;
    } else {
      const uint2 u = make_uint2(pack_bf16x2(pm[0], pm[1]), pack_bf16x2(pm[2], pm[3]));
      if (MODE == RS_NVLS_PUSH) multimem_st_v2(p.p16_mc + i * N, u);
      else *reinterpret_cast<uint2*>(p.p16 + i * N) = u;
    }
  }

  // 3. the last block to finish tells every peer that this rank is done reading their
  //    buckets and that its bf16 shard now holds the parameters of this epoch.
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    if (s_ok && threadIdx.x < p.R) {
      st_release_sys(p.flags[threadIdx.x] + 1 * p.R + p.r, p.epoch);
      st_release_sys(p.flags[threadIdx.x] + 2 * p.R + p.r, p.epoch);
    }
    if (threadIdx.x == 0) *p.counter = 0u;
  }
}

// Default variant.  All loads of an iteration - optimizer state and the R gradient slices of V vectors per thread -
// are issued before anything is consumed, so one NVLink round trip covers them all and a thread keeps V * (R + 6)
// 16-byte requests in flight.  RT bounds R at compile time (register arrays sized for the group, not for 8).
// Same protocol, same summation order (rank 0, 1, ...) and same arithmetic as the generic kernel above.
template <typename GT, int RT, int V>
__global__ void __launch_bounds__(256)
rs_adam_early_kernel(const RsAdamParams p) {
  constexpr int N = GradVec<GT>::N;
  __shared__ int s_ok;
  if (blockIdx.x == 0 && threadIdx.x < p.R) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + 0 * p.R + p.r, p.epoch);
  }
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int q = 0; q < p.R && ok; ++q)
      ok = flag_wait_ge(p.flags[p.r] + 0 * p.R + q, p.epoch, p.wait_ns, p.status, ST_TIMEOUT_FLAG);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  const long nvec = s_ok ? p.shard_n / N : 0;
  const long lo = long(p.r) * p.shard_n;
  const long stride = long(gridDim.x) * blockDim.x;
  for (long i0 = blockIdx.x * long(blockDim.x) + threadIdx.x; i0 < nvec; i0 += stride * V) {
    float pm[V][N], mm[V][N], vv[V][N];
    uint4 raw[V][RT];
    bool on[V];
#pragma unroll
    for (int u = 0; u < V; ++u) {
      const long i = i0 + u * stride;
      on[u] = i < nvec && zb_in_bounds(lo + (i + 1) * N <= long(p.R) * p.shard_n, p.status, 5);
      if (on[u]) {
#pragma unroll
        for (int q = 0; q < RT; ++q)
          if (q < p.R) raw[u][q] = ld_v4_relaxed_sys(static_cast<const GT*>(p.grad[q]) + lo + i * N);
#pragma unroll
        for (int k = 0; k < N; k += 4) {
          *reinterpret_cast<float4*>(pm[u] + k) = *reinterpret_cast<const float4*>(p.master + i * N + k);
          *reinterpret_cast<float4*>(mm[u] + k) = *reinterpret_cast<const float4*>(p.m + i * N + k);
          *reinterpret_cast<float4*>(vv[u] + k) = *reinterpret_cast<const float4*>(p.v + i * N + k);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < V; ++u) {
      const long i = i0 + u * stride;
      if (!on[u]) continue;
      float g[N];
#pragma unroll
      for (int k = 0; k < N; ++k) g[k] = 0.f;
#pragma unroll
      for (int q = 0; q < RT; ++q) {
        if (q < p.R) {
          float t[N];
          GradVec<GT>::unpack(raw[u][q], t);
#pragma unroll
          for (int k = 0; k < N; ++k) g[k] += t[k];
        }
      }
#pragma unroll
      for (int k = 0; k < N; ++k) {
        float gg = g[k] * p.grad_scale;
        if (p.weight_decay != 0.f) gg += p.weight_decay * pm[u][k];
        mm[u][k] = p.beta1 * mm[u][k] + (1.f - p.beta1) * gg;
        vv[u][k] = p.beta2 * vv[u][k] + (1.f - p.beta2) * gg * gg;
        pm[u][k] -= (p.lr / p.bc1) * (mm[u][k] / (sqrtf(vv[u][k]) / p.bc2_sqrt + p.eps));
      }
#pragma unroll
      for (int k = 0; k < N; k += 4) {
        *reinterpret_cast<float4*>(p.master + i * N + k) = *reinterpret_cast<float4*>(pm[u] + k);
        *reinterpret_cast<float4*>(p.m + i * N + k) = *reinterpret_cast<float4*>(mm[u] + k);
        *reinterpret_cast<float4*>(p.v + i * N + k) = *reinterpret_cast<float4*>(vv[u] + k);
      }
      if (N == 8) {
        uint4 o;
        o.x = pack_bf16x2(pm[u][0], pm[u][1]); o.y = pack_bf16x2(pm[u][2], pm[u][3]);
        o.z = pack_bf16x2(pm[u][4], pm[u][5]); o.w = pack_bf16x2(pm[u][6], pm[u][7]);
        *reinterpret_cast<uint4*>(p.p16 + i * N) = o;
      } else {
        *reinterpret_cast<uint2*>(p.p16 + i * N) = make_uint2(pack_bf16x2(pm[u][0], pm[u][1]), pack_bf16x2(pm[u][2], pm[u][3]));
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(p.counter, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    if (s_ok && threadIdx.x < p.R) {
      st_release_sys(p.flags[threadIdx.x] + 1 * p.R + p.r, p.epoch);
      st_release_sys(p.flags[threadIdx.x] + 2 * p.R + p.r, p.epoch);
    }
    if (threadIdx.x == 0) *p.counter = 0u;
  }
}

// Waits until flags[which*R + q] >= epoch for every q (one thread; bounded).
__global__ void wait_flags_kernel(const int* flags, int R, int which, int epoch, unsigned long long wait_ns,
                                  int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    for (int q = 0; q < R; ++q)
      if (!flag_wait_ge(flags + which * R + q, epoch, wait_ns, status, ST_TIMEOUT_FLAG)) break;
  }
}

// Copies `bytes` (multiple of 16) from a peer-mapped pointer into local memory.
__global__ void __launch_bounds__(256)
peer_pull_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long n16) {
  long i = blockIdx.x * long(blockDim.x) + threadIdx.x;
  const long stride = long(gridDim.x) * blockDim.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 a = ld_v4_relaxed_sys(src + i), b = ld_v4_relaxed_sys(src + i + stride),
          c = ld_v4_relaxed_sys(src + i + 2 * stride), d = ld_v4_relaxed_sys(src + i + 3 * stride);
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) dst[i] = ld_v4_relaxed_sys(src + i);
}

}  // namespace zb

static int g_rs_adam_variant = 1;   // 1 = loads issued up front (default), 0 = one peer after another

static int rs_adam_launch(const void* const* grad_ptrs, const void* grad_mc, void* p16_mc, int* const* flag_ptrs, int R, int r,
                          long shard_n, float* master, float* m, float* v, void* p16, float lr, float beta1,
                          float beta2, float eps, float weight_decay, int step, float grad_scale, int grad_f32,
                          int epoch, unsigned int* counter, int max_blocks, double wait_seconds, int* status,
                          cudaStream_t stream) {
  using namespace zb;
  if (R < 1 || R > MAX_R) ZB_FAIL(-1, "rs_adam: group size %d unsupported (1..%d)", R, MAX_R);
  if (shard_n % 8 != 0) ZB_FAIL(-1, "rs_adam: shard size %ld not a multiple of 8", shard_n);
  RsAdamParams p;
  for (int i = 0; i < R; ++i) { p.grad[i] = grad_ptrs ? grad_ptrs[i] : nullptr; p.flags[i] = flag_ptrs[i]; }
  p.grad_mc = grad_mc;
  p.p16_mc = static_cast<__nv_bfloat16*>(p16_mc);
  p.R = R; p.r = r; p.shard_n = shard_n;
  p.master = master; p.m = m; p.v = v; p.p16 = static_cast<__nv_bfloat16*>(p16);
  p.lr = lr; p.beta1 = beta1; p.beta2 = beta2; p.eps = eps; p.weight_decay = weight_decay;
  p.bc1 = 1.f - powf(beta1, float(step));
  p.bc2_sqrt = sqrtf(1.f - powf(beta2, float(step)));
  p.grad_scale = grad_scale;
  p.epoch = epoch; p.status = status; p.counter = counter;
  p.wait_ns = (unsigned long long)(wait_seconds * 1e9);
  // two CTAs per SM: the CTAs spin at their start until every peer has announced its bucket, so
  // they must leave room on each SM for the kernels (NCCL p2p, GEMMs) the peers may still need
  int blocks = num_sms() * 2;
  if (max_blocks > 0 && max_blocks < blocks) blocks = max_blocks;
  long need = (shard_n / (grad_f32 ? 4 : 8) + 255) / 256;
  if (need < blocks) blocks = int(need < 1 ? 1 : need);
  if (grad_mc != nullptr && p16_mc != nullptr) {
    if (grad_f32) rs_adam_kernel<float, RS_NVLS_PUSH><<<blocks, 256, 0, stream>>>(p);
    else rs_adam_kernel<__nv_bfloat16, RS_NVLS_PUSH><<<blocks, 256, 0, stream>>>(p);
  } else if (grad_mc != nullptr) {
    if (grad_f32) rs_adam_kernel<float, RS_NVLS><<<blocks, 256, 0, stream>>>(p);
    else rs_adam_kernel<__nv_bfloat16, RS_NVLS><<<blocks, 256, 0, stream>>>(p);
  } else if (g_rs_adam_variant == 1) {
#define ZB_EARLY(GT_)                                                                              \
    do {                                                                                           \
      if (R <= 2) rs_adam_early_kernel<GT_, 2, 2><<<blocks, 256, 0, stream>>>(p);                  \
      else if (R <= 4) rs_adam_early_kernel<GT_, 4, 2><<<blocks, 256, 0, stream>>>(p);             \
      else rs_adam_early_kernel<GT_, 8, 1><<<blocks, 256, 0, stream>>>(p);                         \
    } while (0)
    if (grad_f32) ZB_EARLY(float);
    else ZB_EARLY(__nv_bfloat16);
#undef ZB_EARLY
  } else {
    if (grad_f32) rs_adam_kernel<float, RS_PLAIN><<<blocks, 256, 0, stream>>>(p);
    else rs_adam_kernel<__nv_bfloat16, RS_PLAIN><<<blocks, 256, 0, stream>>>(p);
  }
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

extern "C" {

// 1 (default) = the optimizer state and all R slices are requested up front; 0 = one peer after another.
void zb_set_rs_adam_variant(int v) { g_rs_adam_variant = v; }

// grad_ptrs / flag_ptrs: host arrays of R device pointers (peer-mapped), ordered by rank in
// the shard group. counter: a zeroed device int owned by the caller.
int zb_rs_adam(const void* const* grad_ptrs, int* const* flag_ptrs, int R, int r, long shard_n, float* master,
               float* m, float* v, void* p16, float lr, float beta1, float beta2, float eps, float weight_decay,
               int step, float grad_scale, int grad_f32, int epoch, unsigned int* counter, int max_blocks,
               double wait_seconds, int* status, cudaStream_t stream) {
  return rs_adam_launch(grad_ptrs, nullptr, nullptr, flag_ptrs, R, r, shard_n, master, m, v, p16, lr, beta1, beta2, eps,
                        weight_decay, step, grad_scale, grad_f32, epoch, counter, max_blocks, wait_seconds, status,
                        stream);
}

// Same update with the gradient slice reduced inside NVSwitch: grad_mc is the multicast address
// of the group's buckets (every rank's bucket bound at the same offset of one multicast object).
// The summation order is the switch's, so results can differ from zb_rs_adam in the last bit.
// p16_mc (optional): multicast address of this rank's shard inside the group's unsharded parameter
// buffers; when given, the refreshed bf16 shard is stored there (reaching every rank) instead of p16.
int zb_rs_adam_nvls(const void* grad_mc, void* p16_mc, int* const* flag_ptrs, int R, int r, long shard_n, float* master, float* m,
                    float* v, void* p16, float lr, float beta1, float beta2, float eps, float weight_decay, int step,
                    float grad_scale, int grad_f32, int epoch, unsigned int* counter, int max_blocks,
                    double wait_seconds, int* status, cudaStream_t stream) {
  if (grad_mc == nullptr || (reinterpret_cast<uintptr_t>(grad_mc) & 15))
    ZB_FAIL(-1, "rs_adam_nvls: no multicast address for the gradient buckets (or not 16-byte aligned)");
  if (reinterpret_cast<uintptr_t>(p16_mc) & 15) ZB_FAIL(-1, "rs_adam_nvls: parameter multicast address not 16-byte aligned");
  return rs_adam_launch(nullptr, grad_mc, p16_mc, flag_ptrs, R, r, shard_n, master, m, v, p16, lr, beta1, beta2, eps,
                        weight_decay, step, grad_scale, grad_f32, epoch, counter, max_blocks, wait_seconds, status,
                        stream);
}

int zb_wait_flags(const int* flags, int R, int which, int epoch, double wait_seconds, int* status,
                  cudaStream_t stream) {
  using namespace zb;
  wait_flags_kernel<<<1, 32, 0, stream>>>(flags, R, which, epoch, (unsigned long long)(wait_seconds * 1e9), status);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

int zb_peer_pull(const void* src, void* dst, long bytes, int max_blocks, cudaStream_t stream) {
  using namespace zb;
  if (bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
    ZB_FAIL(-1, "peer_pull: pointers and size must be multiples of 16 bytes");
  if (bytes <= 0) return 0;
  long n16 = bytes / 16;
  int blocks = num_sms() * 2;
  if (max_blocks > 0 && max_blocks < blocks) blocks = max_blocks;
  long need = (n16 + 1023) / 1024;
  if (need < blocks) blocks = int(need < 1 ? 1 : need);
  peer_pull_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), n16);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
