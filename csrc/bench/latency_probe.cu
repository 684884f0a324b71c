// In-kernel latency / throughput probe for the building blocks the attention and GEMM kernels
// are made of (sm_100a): tcgen05.ld / st round trips, tcgen05.mma issue -> commit -> mbarrier
// observed, mbarrier hand-off between warps, MUFU ex2 and fma issue cost with one and two warps
// per scheduler.  One CTA, clock64 deltas, results in a small global array; the numbers feed
// the pipeline models in the kernel headers.  No counterpart in the reference.
//
// Layout: warps 0-7 are measuring warps (warp w sits on scheduler w % 4), warp 8 issues MMAs.
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

enum : int {
  LP_TMEM_LD32 = 0,        // one tcgen05.ld.32x32b.x32 + wait::ld
  LP_TMEM_LD128 = 1,       // four x32 loads, one wait
  LP_TMEM_ST32 = 2,        // one tcgen05.st.32x32b.x32 + wait::st
  LP_MBAR_HANDOFF = 3,     // arrive (warp 0) -> observed by a spinning warp 1
  LP_MMA_1 = 4,            // issue 1 MMA 128x128x16 + commit -> issuer observes the barrier
  LP_MMA_8 = 5,
  LP_MMA_16 = 6,
  LP_MMA_32 = 7,
  LP_MMA_OBSERVED_BY_OTHER = 8,  // 8 MMAs + commit -> a spinning warp of another scheduler observes
  LP_EX2_1WARP = 9,        // 1024 ex2 per lane, one warp per scheduler: clocks
  LP_EX2_2WARP = 10,       // the same with two warps per scheduler: clocks (of warp 0)
  LP_FMA_1WARP = 11,       // 1024 fma per lane, one warp per scheduler
  LP_FMA_2WARP = 12,
  LP_POLY_1WARP = 13,      // 1024 exp2_poly3 per lane, one warp per scheduler
  LP_COUNT = 16,
};

__global__ void __launch_bounds__(288, 1)
latency_probe_kernel(unsigned long long* __restrict__ out, float* __restrict__ sink, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                 // [128 x 64] bf16, zero
  uint8_t* sB = smem + 16384;         // [128 x 64] bf16, zero
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 32768);   // [0] mma, [1] handoff, [2] mma->other
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile unsigned long long* t_arrive = reinterpret_cast<volatile unsigned long long*>(tmem_slot + 2);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  WaitCtx wctx{abort_flag, status};

  for (int i = threadIdx.x; i < 32768 / 16; i += blockDim.x) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);

  // ---- TMEM round trips (warp 0) ----
  if (warp == 0) {
    uint32_t r[32], r1[32], r2[32], r3[32];
    long long t0 = clock64();
    tmem_ld32(lane_addr, r);
    tmem_wait_ld();
    long long t1 = clock64();
    if (lane == 0) out[LP_TMEM_LD32] = t1 - t0;
    t0 = clock64();
    tmem_ld32(lane_addr, r);
    tmem_ld32(lane_addr + 32u, r1);
    tmem_ld32(lane_addr + 64u, r2);
    tmem_ld32(lane_addr + 96u, r3);
    tmem_wait_ld();
    t1 = clock64();
    if (lane == 0) out[LP_TMEM_LD128] = t1 - t0;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) acc += __uint_as_float(r[k] ^ r1[k] ^ r2[k] ^ r3[k]);
    t0 = clock64();
    tmem_st32(lane_addr, r);
    tmem_wait_st();
    t1 = clock64();
    if (lane == 0) out[LP_TMEM_ST32] = t1 - t0;
    sink[threadIdx.x] = acc;
  }
  __syncthreads();

  // ---- mbarrier hand-off: warp 0 arrives, warp 1 (another scheduler) spins ----
  if (warp == 1) {
    const bool ok = mbar_wait(&bars[1], 0, wctx, ST_TIMEOUT_MISC);
    const long long t1 = clock64();
    if (lane == 0 && ok) out[LP_MBAR_HANDOFF] = static_cast<unsigned long long>(t1) - *t_arrive;
  } else if (warp == 0) {
    for (int i = 0; i < 20; ++i) __nanosleep(100);   // let warp 1 reach its spin loop
    if (lane == 0) {
      *t_arrive = static_cast<unsigned long long>(clock64());
      __threadfence_block();
      mbar_arrive(&bars[1]);
    }
  }
  __syncthreads();

  // ---- MMA issue -> commit -> observed (warp 8 issues; in the last round warp 2 observes) ----
  if (warp == 8 && lane == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, 128, false, false);
    const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
    const int counts[4] = {1, 8, 16, 32};
    uint32_t phase = 0;
    for (int t = 0; t < 4; ++t) {
      const long long t0 = clock64();
      for (int i = 0; i < counts[t]; ++i)
        umma_f16_ss(tmem_base, umma_desc_kmajor(a_addr + uint32_t(i % 4) * 32), umma_desc_kmajor(b_addr + uint32_t(i % 4) * 32),
                    idesc, i != 0 ? 1u : 0u);
      umma_commit(&bars[0]);
      const bool ok = mbar_wait(&bars[0], phase, wctx, ST_TIMEOUT_TMEM_FULL);
      const long long t1 = clock64();
      phase ^= 1;
      if (ok) out[LP_MMA_1 + t] = t1 - t0;
    }
    for (int i = 0; i < 20; ++i) __nanosleep(100);   // let warp 2 reach its spin loop
    *t_arrive = static_cast<unsigned long long>(clock64());
    __threadfence_block();
    for (int i = 0; i < 8; ++i)
      umma_f16_ss(tmem_base, umma_desc_kmajor(a_addr + uint32_t(i % 4) * 32), umma_desc_kmajor(b_addr + uint32_t(i % 4) * 32),
                  idesc, i != 0 ? 1u : 0u);
    umma_commit(&bars[2]);
  } else if (warp == 2) {
    const bool ok = mbar_wait(&bars[2], 0, wctx, ST_TIMEOUT_TMEM_FULL);
    const long long t1 = clock64();
    if (lane == 0 && ok) out[LP_MMA_OBSERVED_BY_OTHER] = static_cast<unsigned long long>(t1) - *t_arrive;
  }
  __syncthreads();

  // ---- issue cost of ex2 / fma / polynomial exp2: 8 independent chains, 1024 ops per lane ----
  auto run_ex2 = [&]() -> float {
    float x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = -0.001f * float(lane + k);
    for (int it = 0; it < 128; ++it) {
#pragma unroll
      for (int k = 0; k < 8; ++k) x[k] = exp2f(x[k]) - 1.0009765625f;
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += x[k];
    return s;
  };
  auto run_fma = [&]() -> float {
    float x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = 0.001f * float(lane + k);
    for (int it = 0; it < 128; ++it) {
#pragma unroll
      for (int k = 0; k < 8; ++k) x[k] = fmaf(x[k], 0.999f, 0.0001f);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += x[k];
    return s;
  };
  auto run_poly = [&]() -> float {
    float x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) x[k] = -0.001f * float(lane + k);
    for (int it = 0; it < 128; ++it) {
#pragma unroll
      for (int k = 0; k < 8; ++k) x[k] = exp2_poly3(x[k]) - 1.0009765625f;
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) s += x[k];
    return s;
  };
  float keep = 0.f;
  // one warp per scheduler: warps 0-3
  if (warp < 4) {
    long long t0 = clock64();
    keep += run_ex2();
    long long t1 = clock64();
    if (threadIdx.x == 0) out[LP_EX2_1WARP] = t1 - t0;
    t0 = clock64();
    keep += run_fma();
    t1 = clock64();
    if (threadIdx.x == 0) out[LP_FMA_1WARP] = t1 - t0;
    t0 = clock64();
    keep += run_poly();
    t1 = clock64();
    if (threadIdx.x == 0) out[LP_POLY_1WARP] = t1 - t0;
  }
  __syncthreads();
  // two warps per scheduler: warps 0-7
  if (warp < 8) {
    long long t0 = clock64();
    keep += run_ex2();
    long long t1 = clock64();
    if (threadIdx.x == 0) out[LP_EX2_2WARP] = t1 - t0;
  }
  __syncthreads();
  if (warp < 8) {
    long long t0 = clock64();
    keep += run_fma();
    long long t1 = clock64();
    if (threadIdx.x == 0) out[LP_FMA_2WARP] = t1 - t0;
  }
  if (warp < 8) sink[threadIdx.x] += keep;

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
}

}  // namespace zb

extern "C" int zb_latency_probe_count() { return zb::LP_COUNT; }

// out: LP_COUNT 64-bit words (zeroed by the caller), sink: 288 floats, status: the status word.
extern "C" int zb_latency_probe(unsigned long long* out, float* sink, int* status, cudaStream_t stream) {
  using namespace zb;
  constexpr int SMEM = 32768 + 1024 + 256;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(latency_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    attr_set = true;
  }
  latency_probe_kernel<<<1, 288, SMEM, stream>>>(out, sink, status);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}
