// Flash attention backward for sm_100a (causal / sliding window / GQA), tcgen05 + TMEM.
//
// One CTA per (batch, kv head, 128-row key/value tile).  K and V stay in shared memory;
// the CTA walks over the query heads of the GQA group and the query tiles that see this
// key tile.  Per (query tile) step, five GEMMs on tcgen05 with fp32 accumulators in TMEM:
//     S  = Q K^T          dP = dO V^T                      (TMEM cols [0,128) / [128,256))
//     dV += P^T dO        dK += dS^T Q                     (TMEM cols [256,256+D) / [256+D,256+2D))
//     dQ = dS K           (reuses the S columns; added to an fp32 accumulator in global
//                          memory with red.global.add.v4.f32, one row per thread)
// Warps 0-7 (0-3: key columns 0-63, 4-7: columns 64-127 of the tile; every warp covers 32 query
// rows) turn S/dP into P and dS = P * (dP - delta) * scale in registers and write both
// as bf16 into 128-byte-swizzled shared tiles whose layout serves as the K-major operand
// of dS K and as the MN-major operand of P^T dO / dS^T Q.  dK and dV never leave TMEM
// until the CTA is done, so no atomics are needed for them.
//
// Inputs: packed qkv[B*S, (Hq+2Hkv)*D], O and dO [B*S, Hq*D], LSE[B,Hq,S].
// Outputs: dqkv (k and v parts written here, q part by attn_dq_finish_kernel from the fp32
// accumulator).  Warp 8 = TMA producer, warp 9 = MMA issuer and TMEM owner.  Replaces the autograd of flash-attn 2 / SDPA used by the reference
// (models/llama_simple.py:396-416).
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "attn_bwd_common.h"

namespace zb {

template <int D>
struct AttnBwdCfg {
  static constexpr int BM = 128, BN = 128;
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int QS = (D == 64) ? 2 : 1;  // Q / dO stages
  static constexpr int PS_BYTES = 128 * 128 * 2;
  static constexpr int SMEM_BYTES = 2 * TILE_BYTES + QS * 2 * TILE_BYTES + 2 * PS_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int DP_COL = 128, DV_COL = 256, DK_COL = 256 + D;
};

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <int D>
__global__ void __launch_bounds__(320, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                 const AttnBwdParams p) {
  using Cfg = AttnBwdCfg<D>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, QS = Cfg::QS, DB = D / 64;
  constexpr int BLK = 128 * 128;  // bytes of one [128 rows x 64 cols] block
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::TILE_BYTES;
  uint8_t* sQ = sV + Cfg::TILE_BYTES;
  uint8_t* sDO = sQ + QS * Cfg::TILE_BYTES;
  uint8_t* sP = sDO + QS * Cfg::TILE_BYTES;
  uint8_t* sDS = sP + Cfg::PS_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + Cfg::PS_BYTES);
  uint64_t* kv_full = bars;            // 1
  uint64_t* qdo_full = bars + 1;       // QS
  uint64_t* qdo_empty = qdo_full + 2;  // QS
  uint64_t* sdp_full = qdo_empty + 2;  // 1
  uint64_t* pds_full = sdp_full + 1;   // 1 (8 arrivals)
  uint64_t* dq_full = pds_full + 1;    // 1
  uint64_t* dq_empty = dq_full + 1;    // 1 (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x, kv_head = blockIdx.y, batch = blockIdx.z;
  const int kv0 = jt * BN;
  const int rep = p.Hq / p.Hkv;
  const int n_qt = (p.S + BM - 1) / BM;
  const int i_lo = p.causal ? (kv0 / BM) : 0;
  int i_hi = n_qt;
  if (p.window > 0) i_hi = min(n_qt, (kv0 + BN - 1 + p.window - 1) / BM + 1);
  const int per_head = max(i_hi - i_lo, 0);
  const int n_iters = per_head * rep;
  WaitCtx wctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    for (int i = 0; i < QS; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 8);
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(kv_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
      for (int b = 0; b < DB; ++b) {
        tma_load_4d(sK + b * BLK, &tmap_k, kv_full, b * 64, kv_head, kv0, batch);
        tma_load_4d(sV + b * BLK, &tmap_v, kv_full, b * 64, kv_head, kv0, batch);
      }
      for (int it = 0; it < n_iters; ++it) {
        const int st = it % QS;
        const uint32_t ph = uint32_t(it / QS) & 1;
        const int head = kv_head * rep + it / per_head;
        const int q0 = (i_lo + it % per_head) * BM;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&qdo_full[st], 2 * Cfg::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_4d(sQ + st * Cfg::TILE_BYTES + b * BLK, &tmap_q, &qdo_full[st], b * 64, head, q0, batch);
          tma_load_4d(sDO + st * Cfg::TILE_BYTES + b * BLK, &tmap_do, &qdo_full[st], b * 64, head, q0, batch);
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_iters > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_dkv = umma_idesc_bf16(128, D, true, true);
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, D, false, true);
      bool ok = mbar_wait(kv_full, 0, wctx, ST_TIMEOUT_FULL);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), p_addr = smem_u32(sP), ds_addr = smem_u32(sDS);
      for (int it = 0; it < n_iters && ok; ++it) {
        const int st = it % QS;
        const uint32_t ph = uint32_t(it / QS) & 1;
        const uint32_t q_addr = smem_u32(sQ + st * Cfg::TILE_BYTES), do_addr = smem_u32(sDO + st * Cfg::TILE_BYTES);
        if (!mbar_wait(&qdo_full[st], ph, wctx, ST_TIMEOUT_FULL)) break;
        if (it > 0 && !mbar_wait(dq_empty, uint32_t(it - 1) & 1, wctx, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
          umma_f16_ss(tmem_base, umma_desc_kmajor(q_addr + off), umma_desc_kmajor(k_addr + off), idesc_s,
                      kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
          umma_f16_ss(tmem_base + Cfg::DP_COL, umma_desc_kmajor(do_addr + off), umma_desc_kmajor(v_addr + off),
                      idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
        if (!mbar_wait(pds_full, uint32_t(it) & 1, wctx, ST_TIMEOUT_MISC)) break;
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q   (reduction over the 128 query rows)
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {
          umma_f16_ss(tmem_base + Cfg::DV_COL, umma_desc_mnmajor(p_addr + kk * 2048, BLK),
                      umma_desc_mnmajor(do_addr + kk * 2048, BLK), idesc_dkv, (it | kk) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {
          umma_f16_ss(tmem_base + Cfg::DK_COL, umma_desc_mnmajor(ds_addr + kk * 2048, BLK),
                      umma_desc_mnmajor(q_addr + kk * 2048, BLK), idesc_dkv, (it | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&qdo_empty[st]);
        // dQ = dS K   (reduction over the 128 keys) into the S columns
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t aoff = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
          umma_f16_ss(tmem_base, umma_desc_kmajor(ds_addr + aoff), umma_desc_mnmajor(k_addr + kk * 2048, BLK),
                      idesc_dq, kk != 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
      }
    }
  } else {
    // ------------------------------ softmax-grad warps ------------------------------
    // warps 0-3 take columns [0,64) of S / dP (and the first half of the dQ, dK, dV columns),
    // warps 4-7 the other half; both sets cover TMEM lanes (= rows) 0..127
    const int half = warp >> 2;
    const int t = (warp & 3) * 32 + lane;  // row within the query tile (steps) / key tile (final write)
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    bool ok = true;
    for (int it = 0; it < n_iters; ++it) {
      const int head = kv_head * rep + it / per_head;
      const int q0 = (i_lo + it % per_head) * BM;
      const int row = q0 + t;
      const bool row_ok = row < p.S;
      float lse_r = 0.f, delta_r = 0.f;
      if (row_ok) {
        const size_t si = (size_t(batch) * p.Hq + head) * p.S + row;
        lse_r = p.lse[si] * LOG2E;
        delta_r = p.delta[si];
      }
      if (!__all_sync(0xffffffffu, mbar_wait(sdp_full, uint32_t(it) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (p.causal && kv0 + BN - 1 > q0) || (p.window > 0 && kv0 < q0 + BM - p.window) ||
                             (kv0 + BN > p.S) || (q0 + BM > p.S);
      uint8_t* prow = sP + t * 128;
      uint8_t* dsrow = sDS + t * 128;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t rs[32], rd[32];
        tmem_ld32(lane_addr + uint32_t(c * 32), rs);
        tmem_ld32(lane_addr + uint32_t(Cfg::DP_COL + c * 32), rd);
        tmem_wait_ld();
        float pv[32], dsv[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          float pe = exp2f(fmaf(__uint_as_float(rs[k]), p.scale_log2, -lse_r));
          if (need_mask) {
            const int col = kv0 + c * 32 + k;
            const bool vis = row_ok && (col < p.S) && (!p.causal || col <= row) &&
                             (p.window <= 0 || row - col < p.window);
            pe = vis ? pe : 0.f;
          }
          pv[k] = pe;
          dsv[k] = pe * (__uint_as_float(rd[k]) - delta_r) * p.scale;
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint4 up, ud;
          up.x = pack_bf16x2(pv[v4 * 8 + 0], pv[v4 * 8 + 1]); up.y = pack_bf16x2(pv[v4 * 8 + 2], pv[v4 * 8 + 3]);
          up.z = pack_bf16x2(pv[v4 * 8 + 4], pv[v4 * 8 + 5]); up.w = pack_bf16x2(pv[v4 * 8 + 6], pv[v4 * 8 + 7]);
          ud.x = pack_bf16x2(dsv[v4 * 8 + 0], dsv[v4 * 8 + 1]); ud.y = pack_bf16x2(dsv[v4 * 8 + 2], dsv[v4 * 8 + 3]);
          ud.z = pack_bf16x2(dsv[v4 * 8 + 4], dsv[v4 * 8 + 5]); ud.w = pack_bf16x2(dsv[v4 * 8 + 6], dsv[v4 * 8 + 7]);
          const int chunk = c * 4 + v4;  // 16-byte chunk index within the 128-key row
          const int blk = chunk >> 3, ch = chunk & 7;
          const int soff = blk * BLK + ((ch ^ (t & 7)) << 4);
          *reinterpret_cast<uint4*>(prow + soff) = up;
          *reinterpret_cast<uint4*>(dsrow + soff) = ud;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      // dQ tile -> global fp32 accumulator
      if (!__all_sync(0xffffffffu, mbar_wait(dq_full, uint32_t(it) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tc_fence_after();
      float* dq_row = p.dq_acc + (size_t(batch) * p.S + row) * (size_t(p.Hq) * D) + size_t(head) * D;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t r[32];
        tmem_ld32(lane_addr + uint32_t(c * 32), r);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int v4 = 0; v4 < 8; ++v4)
            red_add_v4(dq_row + c * 32 + v4 * 4, __uint_as_float(r[v4 * 4 + 0]), __uint_as_float(r[v4 * 4 + 1]),
                       __uint_as_float(r[v4 * 4 + 2]), __uint_as_float(r[v4 * 4 + 3]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);
    }
    // ------------------------------ dK / dV write-out ------------------------------
    // the last dq_full arrival also covers every dK / dV MMA issued before it
    const int krow = kv0 + t;
    const int width = (p.Hq + 2 * p.Hkv) * D;
    ok = __all_sync(0xffffffffu, ok);
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const uint32_t col0 = which == 0 ? Cfg::DK_COL : Cfg::DV_COL;
      __nv_bfloat16* dst = p.dqkv + (size_t(batch) * p.S + krow) * width +
                           size_t(which == 0 ? (p.Hq + kv_head) : (p.Hq + p.Hkv + kv_head)) * D;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t r[32];
        if (n_iters > 0) {
          tmem_ld32(lane_addr + col0 + uint32_t(c * 32), r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) r[k] = 0u;
        }
        if (ok && krow < p.S) {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(r[v4 * 8 + 0]), __uint_as_float(r[v4 * 8 + 1]));
            u.y = pack_bf16x2(__uint_as_float(r[v4 * 8 + 2]), __uint_as_float(r[v4 * 8 + 3]));
            u.z = pack_bf16x2(__uint_as_float(r[v4 * 8 + 4]), __uint_as_float(r[v4 * 8 + 5]));
            u.w = pack_bf16x2(__uint_as_float(r[v4 * 8 + 6]), __uint_as_float(r[v4 * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + v4 * 8) = u;
          }
        }
      }
    }
  }

  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// delta[b, h, s] = sum_d dO * O ; one warp per (token, head)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int S, int Hq, int D) {
  const long wid = (blockIdx.x * long(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = long(B) * S * Hq;
  if (wid >= total) return;
  const int h = int(wid % Hq);
  const long tok = wid / Hq;
  const __nv_bfloat16* po = o + tok * (long(Hq) * D) + long(h) * D;
  const __nv_bfloat16* pd = d_o + tok * (long(Hq) * D) + long(h) * D;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(po + c));
    float2 b = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(pd + c));
    acc += a.x * b.x + a.y * b.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long b = tok / S, s = tok % S;
    delta[(b * Hq + h) * S + s] = acc;
  }
}

// dqkv[:, :Hq*D] = bf16(dq_acc); dq_acc is cleared for the next call.
__global__ void attn_dq_finish_kernel(float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, long T, int qw,
                                      int width) {
  const int cpr = qw >> 3;
  const long total = T * cpr;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const long t = i / cpr;
    const int c = int(i % cpr);
    float4* src = reinterpret_cast<float4*>(dq_acc + t * qw + c * 8);
    float4 a = src[0], b = src[1];
    uint4 u;
    u.x = pack_bf16x2(a.x, a.y); u.y = pack_bf16x2(a.z, a.w);
    u.z = pack_bf16x2(b.x, b.y); u.w = pack_bf16x2(b.z, b.w);
    *reinterpret_cast<uint4*>(dqkv + t * width + c * 8) = u;
    src[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    src[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

int attn_bwd_delta(const __nv_bfloat16* o, const __nv_bfloat16* d_o, float* delta, int B, int S, int Hq, int D,
                   cudaStream_t stream) {
  const long warps = long(B) * S * Hq;
  const int threads = 256;
  const long blocks = (warps * 32 + threads - 1) / threads;
  attn_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>(o, d_o, delta, B, S, Hq, D);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

int attn_bwd_finish_dq(float* dq_acc, __nv_bfloat16* dqkv, int B, int S, int Hq, int Hkv, int D, cudaStream_t stream) {
  const long T = long(B) * S;
  const int qw = Hq * D, width = (Hq + 2 * Hkv) * D;
  long blocks = (T * (qw / 8) + 255) / 256;
  long cap = long(num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  attn_dq_finish_kernel<<<(unsigned)blocks, 256, 0, stream>>>(dq_acc, dqkv, T, qw, width);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

static int make_head_tmap_bwd(CUtensorMap* out, const __nv_bfloat16* base, int B, int S, int heads, int D, int width) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(heads), uint64_t(S), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(width) * 2, uint64_t(width) * 2 * uint64_t(S)};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_nd_bf16(out, base, 4, dims, strides, box);
}

template <int D>
static int launch_bwd(const __nv_bfloat16* qkv, const __nv_bfloat16* d_o, const AttnBwdParams& p, cudaStream_t stream) {
  using Cfg = AttnBwdCfg<D>;
  const int width = (p.Hq + 2 * p.Hkv) * D;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_head_tmap_bwd(&tq, qkv, p.B, p.S, p.Hq, D, width))) return rc;
  if ((rc = make_head_tmap_bwd(&tk, qkv + size_t(p.Hq) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  if ((rc = make_head_tmap_bwd(&tv, qkv + size_t(p.Hq + p.Hkv) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  if ((rc = make_head_tmap_bwd(&tdo, d_o, p.B, p.S, p.Hq, D, p.Hq * D))) return rc;
  auto kern = flash_bwd_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set = true;
  }
  dim3 grid((p.S + 127) / 128, p.Hkv, p.B);
  kern<<<grid, 320, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, p);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace zb

extern "C" {

// Scratch: delta fp32 [B*Hq*S]; dq_acc fp32 [B*S*Hq*D], zero on entry (left zero on exit).
int zb_flash_bwd(const void* d_o, const void* qkv, const void* o, const float* lse, void* dqkv, float* delta,
                 float* dq_acc, int B, int S, int Hq, int Hkv, int D, int causal, int window, float softmax_scale,
                 int* status, cudaStream_t stream) {
  using namespace zb;
  if (B <= 0 || S <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) ZB_FAIL(-1, "attention: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  if (D != 64 && D != 128) ZB_FAIL(-1, "attention: head dim %d unsupported (64 or 128)", D);
  auto DO = static_cast<const __nv_bfloat16*>(d_o);
  auto O = static_cast<const __nv_bfloat16*>(o);
  auto QKV = static_cast<const __nv_bfloat16*>(qkv);
  if (int rc = attn_bwd_delta(O, DO, delta, B, S, Hq, D, stream)) return rc;
  AttnBwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.window = window; p.causal = causal;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  int rc = (D == 128) ? launch_bwd<128>(QKV, DO, p, stream) : launch_bwd<64>(QKV, DO, p, stream);
  if (rc) return rc;
  return attn_bwd_finish_dq(dq_acc, p.dqkv, B, S, Hq, Hkv, D, stream);
}

}  // extern "C"
