// Flash attention backward, query-gradient half (sm_100a, tcgen05 + TMEM).
//
// The backward pass is split in two kernels so that neither needs atomics: the key-tile kernel
// (flash_bwd2.cu built without its dQ part) accumulates dK and dV of one key tile in tensor memory
// while it walks over the query tiles, and this kernel accumulates dQ of one query tile in tensor
// memory while it walks over the key tiles.  Scores and dP are formed twice (7 products per tile
// pair instead of 5); in exchange the 4 bytes x 32 adds per dQ element that the one-kernel form
// sends through the L2 atomic units (the measured bound of that form: about 8 k of its 13 k clocks
// per step) disappear, together with the fp32 accumulator and the pass that converts it.
//
// One CTA per (batch, head, 128-row query tile); Q and dO stay in shared memory, K and V tiles
// stream through two rings (K is held until the step's last product, V only until dP).  Per key tile j:
//     S_j  = Q K_j^T            SS  -> TMEM S[j & 1]  (two buffers)
//     dP_j = dO V_j^T           SS  -> TMEM dP
//     P = exp2(S c - lse),  dS = P (dP - delta) scale        compute warps, one query row per thread
//     bf16 dS over the first 32 columns of each 64-column half of S[j & 1]
//     dQ  += dS K_j             TS (A = dS from TMEM)  -> TMEM dQ
// The issuer queues S_{j+1} before it waits for dS_j, so the exponentials of tile j + 1 can start
// while dQ_j and dP_{j+1} run.  lse and delta belong to the thread's own row: loaded once.
//
// Warps 0-7: compute (0-3: key columns 0-63 of the tile, 4-7: columns 64-127; each warp covers 32
// query rows = TMEM lanes), warp 8: TMA producer, warp 9: MMA issuer + TMEM owner.
// TMEM: S0 [0,128) S1 [128,256) dP [256,384) dQ [384, 384+D).
// Replaces (with flash_bwd2.cu) the autograd of flash-attn 2 / SDPA used by the reference
// (models/llama_simple.py:396-416).
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "attn_bwd_common.h"

namespace zb {

template <int D>
struct AttnDqCfg {
  static constexpr int TILE_BYTES = 128 * D * 2;
  // K_j is read by S_j (early) and by dQ_j (the step's last product), V_j only by dP_j: separate rings, the
  // K ring one stage deeper, so that a tile's refill has a whole step to arrive
  static constexpr int NK = (D == 128) ? 3 : 4;
  static constexpr int NV = (D == 128) ? 2 : 3;
  static constexpr int SMEM_BYTES = (2 + NK + NV) * TILE_BYTES + 1024 + 256;
  static constexpr int DP_COL = 256, DQ_COL = 384;
};

template <int D>
__global__ void __launch_bounds__(320, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                    const AttnBwdParams p, const float* __restrict__ stats, int s_pad) {
  using Cfg = AttnDqCfg<D>;
  constexpr int BM = 128, BN = 128, NK = Cfg::NK, NV = Cfg::NV, DB = D / 64;
  constexpr int BLK = 128 * 128;  // bytes of one [128 rows x 64 cols] bf16 block
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + Cfg::TILE_BYTES;
  uint8_t* sK = sDO + Cfg::TILE_BYTES;                // NK tiles
  uint8_t* sV = sK + NK * Cfg::TILE_BYTES;            // NV tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NV * Cfg::TILE_BYTES);
  uint64_t* qdo_full = bars;                 // 1
  uint64_t* k_full = bars + 1;               // NK
  uint64_t* k_empty = k_full + NK;           // NK
  uint64_t* v_full = k_empty + NK;           // NV
  uint64_t* v_empty = v_full + NV;           // NV
  uint64_t* s_full = v_empty + NV;           // 2
  uint64_t* dp_full = s_full + 2;            // 1
  uint64_t* ds_ready = dp_full + 1;          // 1 (8 arrivals)
  uint64_t* dq_done = ds_ready + 1;          // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + BM - 1) / BM;
  // grid = (heads, query tiles, batch): x-fastest dispatch, the latest (heaviest under a causal mask)
  // query tile of every head first
  const int qt = n_qt - 1 - int(blockIdx.y);
  const int head = blockIdx.x, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qt * BM;
  const int n_kv = (p.S + BN - 1) / BN;
  int j_lo = 0, j_hi = n_kv;
  if (p.causal) j_hi = min(j_hi, (q0 + BM - 1) / BN + 1);
  if (p.window > 0) j_lo = max(0, (q0 - p.window + 1) / BN);
  const int n = max(j_hi - j_lo, 0);
  WaitCtx wctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(qdo_full, 1);
    for (int i = 0; i < NK; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < NV; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1);
    mbar_init(ds_ready, 8);
    mbar_init(dq_done, 1);
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && n > 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      tma_prefetch_desc(&tmap_do);
      mbar_expect_tx(qdo_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
      for (int b = 0; b < DB; ++b) {
        tma_load_4d(sQ + b * BLK, &tmap_q, qdo_full, b * 64, head, q0, batch);
        tma_load_4d(sDO + b * BLK, &tmap_do, qdo_full, b * 64, head, q0, batch);
      }
      for (int i = 0; i < n; ++i) {
        const int ks = i % NK, vs = i % NV;
        const int kv0 = (j_lo + i) * BN;
        if (!zb_in_bounds(kv0 >= 0 && kv0 < p.S && q0 < p.S && kv_head < p.Hkv && batch < p.B, p.status, 8)) break;
        if (!mbar_wait(&k_empty[ks], (uint32_t(i / NK) & 1) ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&k_full[ks], Cfg::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          tma_load_4d(sK + ks * Cfg::TILE_BYTES + b * BLK, &tmap_k, &k_full[ks], b * 64, kv_head, kv0, batch);
        if (!mbar_wait(&v_empty[vs], (uint32_t(i / NV) & 1) ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&v_full[vs], Cfg::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          tma_load_4d(sV + vs * Cfg::TILE_BYTES + b * BLK, &tmap_v, &v_full[vs], b * 64, kv_head, kv0, batch);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BM, BN, false, false);   // K-major A and B
      constexpr uint32_t idesc_dq = umma_idesc_bf16(BM, D, false, true);    // A from TMEM, B = K tile [keys][d] (N-major)
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sDO);
      auto k_of = [&](int i) { return smem_u32(sK + (i % NK) * Cfg::TILE_BYTES); };
      auto v_of = [&](int i) { return smem_u32(sV + (i % NV) * Cfg::TILE_BYTES); };
      auto issue_s = [&](int i) {    // S_i = Q K_i^T into S[i & 1]
        const uint32_t k_addr = k_of(i);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
          umma_f16_ss(tmem_base + uint32_t((i & 1) * 128), umma_desc_kmajor(q_addr + off), umma_desc_kmajor(k_addr + off),
                      idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[i & 1]);
      };
      auto issue_dp = [&](int i) {   // dP_i = dO V_i^T
        const uint32_t v_addr = v_of(i);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
          umma_f16_ss(tmem_base + Cfg::DP_COL, umma_desc_kmajor(do_addr + off), umma_desc_kmajor(v_addr + off), idesc_s,
                      kk != 0 ? 1u : 0u);
        }
        umma_commit(dp_full);
        umma_commit(&v_empty[i % NV]);     // dP_i is V_i's only reader
      };
      bool ok = mbar_wait(qdo_full, 0, wctx, ST_TIMEOUT_FULL);
      if (ok) ok = mbar_wait(&k_full[0], 0, wctx, ST_TIMEOUT_FULL);
      if (ok) ok = mbar_wait(&v_full[0], 0, wctx, ST_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      for (int i = 0; i < n && ok; ++i) {
        if (i + 1 < n) {
          if (!mbar_wait(&k_full[(i + 1) % NK], uint32_t((i + 1) / NK) & 1, wctx, ST_TIMEOUT_FULL)) break;
          tc_fence_after();
          issue_s(i + 1);            // its buffer last held dS_{i-1}, consumed by the dQ product queued before this
        }
        if (!mbar_wait(ds_ready, uint32_t(i) & 1, wctx, ST_TIMEOUT_MISC)) break;
        tc_fence_after();
        // dQ += dS_i K_i (reduction over the 128 keys; the bf16 A operand sits in the first 32 columns of each
        // 64-column half of S[i & 1])
        const uint32_t k_addr = k_of(i);
        const uint32_t s_col = tmem_base + uint32_t((i & 1) * 128);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t acol = uint32_t(kk / 4) * 64 + uint32_t(kk % 4) * 8;
          umma_f16_ts(tmem_base + Cfg::DQ_COL, s_col + acol, umma_desc_mnmajor(k_addr + kk * 2048, BLK), idesc_dq,
                      (i | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[i % NK]);     // S_i (queued earlier) and dQ_i are K_i's readers
        if (i + 1 < n) {
          if (!mbar_wait(&v_full[(i + 1) % NV], uint32_t((i + 1) / NV) & 1, wctx, ST_TIMEOUT_FULL)) break;
          tc_fence_after();
          issue_dp(i + 1);                 // the compute warps had dP_i in registers before they announced dS_i
        } else {
          umma_commit(dq_done);
        }
      }
    }
  } else {
    // ------------------------------ compute warps ------------------------------
    const int half = warp >> 2;                  // which 64 key columns of S / dP, which half of the dQ columns
    const int t = (warp & 3) * 32 + lane;        // query row inside the tile = TMEM lane
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const int row = q0 + t;
    const bool row_ok = row < p.S;
    float lse_r = 0.f, delta_r = 0.f;
    if (row_ok) {
      const float* st_row = stats + (size_t(batch) * p.Hq + head) * 2 * size_t(s_pad);
      lse_r = st_row[row];                       // already in log2 units
      delta_r = st_row[s_pad + row];
    }
    bool ok = true;
    for (int i = 0; i < n; ++i) {
      const int kv0 = (j_lo + i) * BN;
      const uint32_t s_col = lane_addr + uint32_t((i & 1) * 128 + half * 64);
      const bool need_mask = (p.causal && kv0 + BN - 1 > q0) || (p.window > 0 && kv0 < q0 + BM - p.window) ||
                             (kv0 + BN > p.S) || (q0 + BM > p.S);
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[i & 1], uint32_t(i >> 1) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tc_fence_after();
      float pr[64];
      {
        // both 32-column chunks in flight before the first is used; the mask test is hoisted out of the
        // element loops (one branch per tile, not per element)
        uint32_t rs0[32], rs1[32];
        tmem_ld32(s_col, rs0);
        tmem_ld32(s_col + 32u, rs1);
        tmem_wait_ld();
        const float nl = -lse_r;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          pr[k] = exp2f(fmaf(__uint_as_float(rs0[k]), p.scale_log2, nl));
          pr[32 + k] = exp2f(fmaf(__uint_as_float(rs1[k]), p.scale_log2, nl));
        }
        if (need_mask) {
          const int col0 = kv0 + half * 64;
#pragma unroll
          for (int k = 0; k < 64; ++k) {
            const int col = col0 + k;
            const bool vis = row_ok && (col < p.S) && (!p.causal || col <= row) && (p.window <= 0 || row - col < p.window);
            pr[k] = vis ? pr[k] : 0.f;
          }
        }
      }
      if (!__all_sync(0xffffffffu, mbar_wait(dp_full, uint32_t(i) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t rd0[32], rd1[32];
        tmem_ld32(lane_addr + uint32_t(Cfg::DP_COL + half * 64), rd0);
        tmem_ld32(lane_addr + uint32_t(Cfg::DP_COL + half * 64 + 32), rd1);
        tmem_wait_ld();
        uint32_t ds0[16], ds1[16];
        // dS = P (dP - delta) scale = (P scale) dP - (P scale) delta: one multiply and one fma per element
        const float nd = -delta_r;
#pragma unroll
        for (int k = 0; k < 32; k += 2) {
          const float a0 = pr[k] * p.scale, a1 = pr[k + 1] * p.scale;
          const float b0 = pr[32 + k] * p.scale, b1 = pr[32 + k + 1] * p.scale;
          ds0[k >> 1] = pack_bf16x2(a0 * (__uint_as_float(rd0[k]) + nd), a1 * (__uint_as_float(rd0[k + 1]) + nd));
          ds1[k >> 1] = pack_bf16x2(b0 * (__uint_as_float(rd1[k]) + nd), b1 * (__uint_as_float(rd1[k + 1]) + nd));
        }
        // packed bf16 over this half's own first 32 columns: the other half's threads only touch their own 64
        tmem_st16(s_col, ds0);
        tmem_st16(s_col + 16u, ds1);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    // ------------------------------ dQ write-out ------------------------------
    if (ok && n > 0) ok = mbar_wait(dq_done, 0, wctx, ST_TIMEOUT_MISC);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    const int width = (p.Hq + 2 * p.Hkv) * D;
    __nv_bfloat16* dst = p.dqkv + (size_t(batch) * p.S + row) * width + size_t(head) * D;
#pragma unroll 1
    for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
      uint32_t r[32];
      if (n > 0) {
        tmem_ld32(lane_addr + uint32_t(Cfg::DQ_COL + c * 32), r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) r[k] = 0u;
      }
      if (ok && row_ok) {
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

  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static int make_head_tmap_dq(CUtensorMap* out, const __nv_bfloat16* base, int B, int S, int heads, int D, int width) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(heads), uint64_t(S), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(width) * 2, uint64_t(width) * 2 * uint64_t(S)};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_nd_bf16(out, base, 4, dims, strides, box);
}

template <int D>
static int launch_dq(const __nv_bfloat16* qkv, const __nv_bfloat16* d_o, const AttnBwdParams& p, const float* stats,
                     int s_pad, cudaStream_t stream) {
  using Cfg = AttnDqCfg<D>;
  const int width = (p.Hq + 2 * p.Hkv) * D;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_head_tmap_dq(&tq, qkv, p.B, p.S, p.Hq, D, width))) return rc;
  if ((rc = make_head_tmap_dq(&tk, qkv + size_t(p.Hq) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  if ((rc = make_head_tmap_dq(&tv, qkv + size_t(p.Hq + p.Hkv) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  if ((rc = make_head_tmap_dq(&tdo, d_o, p.B, p.S, p.Hq, D, p.Hq * D))) return rc;
  auto kern = flash_bwd_dq_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set = true;
  }
  dim3 grid(p.Hq, (p.S + 127) / 128, p.B);
  kern<<<grid, 320, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, p, stats, s_pad);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

// dQ part of the two-kernel backward: writes the q columns of dqkv.  `stats` as written by the key-tile
// kernel's statistics pass (lse in log2 units and delta per row, rows padded to s_pad).
int attn_bwd_dq(const __nv_bfloat16* qkv, const __nv_bfloat16* d_o, const AttnBwdParams& p, const float* stats, int s_pad,
                int D, cudaStream_t stream) {
  if (D == 128) return launch_dq<128>(qkv, d_o, p, stats, s_pad, stream);
  return launch_dq<64>(qkv, d_o, p, stats, s_pad, stream);
}

}  // namespace zb
