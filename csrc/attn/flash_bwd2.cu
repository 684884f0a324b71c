// Flash attention backward, transposed-score formulation (sm_100a, tcgen05 + TMEM).
// Same interface, scratch buffers and memory layouts as flash_bwd.cu.
//
// One CTA per (batch, kv head, 128-key tile); K and V stay in shared memory, Q / dO tiles of the
// query heads of the GQA group stream through TWO shared-memory stages.  Scores are computed
// transposed, keys on the TMEM lanes, so that P^T and dS^T feed the dV / dK products straight
// from tensor memory:
//     A  S^T  = K Q^T             SS   -> R_S  [0,128)      (columns = queries)
//     B  dP^T = V dO^T            SS   -> R_dP [128,256)
//     C  P^T = exp2(S^T c - lse_q), dS^T = P^T (dP^T - delta_q) scale
//        bf16 P^T over R_S, bf16 dS^T over R_dP, dS^T also to shared memory
//     D  dV += P^T dO             TS (A = P^T from TMEM)     -> [256, 256+D)
//     E  dK += dS^T Q             TS (A = dS^T from TMEM)    -> [256+D, 256+2D)
//     F  dQ  = dS K               SS (A = dS^T tile in shared memory, M-major) -> R_dP again
//     G  dQ -> fp32 accumulator in global memory (red.global.add.v4.f32, one query row per thread)
// The issuer queues D E F of step i and A of step i+1 back to back (the tensor pipe runs in
// issue order, so A(i+1) may overwrite R_S right behind D(i)); only B(i+1) waits until G(i) has
// drained dQ out of R_dP.  The compute warps start the exponentials of step i+1 (needs S^T only)
// while B(i+1) is still running.
//
// Warps 0-7: compute (0-3: query columns 0-63, 4-7: columns 64-127; each warp covers 32 key
// lanes), warp 8: TMA producer, warp 9: MMA issuer + TMEM owner.
// With TRACE the first `trace_ctas` CTAs record (clock64, code) per warp at phase boundaries.
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "attn_bwd_common.h"

namespace zb {

constexpr int BWD2_WARPS = 10;
constexpr int BWD2_TRACE_EV = 256;

template <int D>
struct AttnBwd2Cfg {
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int QS = 2;                      // Q / dO stages
  static constexpr int DS_BYTES = 128 * 128 * 2;
  static constexpr int SMEM_BYTES = 2 * TILE_BYTES + QS * 2 * TILE_BYTES + DS_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;
  static constexpr int DP_COL = 128, DV_COL = 256, DK_COL = 256 + D;
};

enum : int {
  TB_S_READY = 1, TB_P_DONE = 2, TB_DP_READY = 3, TB_DS_DONE = 4, TB_DQ_READY = 5, TB_DQ_DRAINED = 6,
  TB_MMA_QDO_READY = 16, TB_MMA_PDS_READY = 17, TB_MMA_DEF_ISSUED = 18, TB_MMA_A_ISSUED = 19, TB_MMA_DQ_EMPTY = 20,
  TB_MMA_B_ISSUED = 21,
  TB_TMA_STAGE_FREE = 32, TB_TMA_ISSUED = 33,
};

__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

__device__ __forceinline__ void red_add_f32(float* p, float a) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(a) : "memory");
}

// DQ = false: the key-tile half of the two-kernel backward (dK and dV only): no dS^T copy in shared memory,
// no dQ product and no atomics; dQ then comes from flash_bwd_dq.cu.
template <int D, bool TRACE, bool DQ>
__global__ void __launch_bounds__(32 * BWD2_WARPS, 1)
flash_bwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                  const AttnBwdParams p, const float* __restrict__ stats, int s_pad,
                  unsigned long long* trace, int trace_ctas) {
  using Cfg = AttnBwd2Cfg<D>;
  constexpr int BM = 128, BN = 128, QS = Cfg::QS, DB = D / 64;
  constexpr int BLK = 128 * 128;  // bytes of one [128 rows x 64 cols] bf16 block
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::TILE_BYTES;
  uint8_t* sQ = sV + Cfg::TILE_BYTES;                 // QS tiles
  uint8_t* sDO = sQ + QS * Cfg::TILE_BYTES;           // QS tiles
  uint8_t* sDS = sDO + QS * Cfg::TILE_BYTES;          // dS^T: [128 keys][128 queries], two 64-query blocks
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + Cfg::DS_BYTES);
  uint64_t* kv_full = bars;             // 1
  uint64_t* qdo_full = bars + 1;        // QS
  uint64_t* qdo_empty = qdo_full + QS;  // QS
  uint64_t* s_full = qdo_empty + QS;    // 1
  uint64_t* dp_full = s_full + 1;       // 1
  uint64_t* pds_full = dp_full + 1;     // 1 (8 arrivals)
  uint64_t* dq_full = pds_full + 1;     // 1
  uint64_t* dq_empty = dq_full + 1;     // 1 (8 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid = (kv heads, key tiles, batch): x-fastest dispatch starts every head's heaviest key tile
  // (tile 0 sees all query tiles under a causal mask) before any light one
  const int jt = blockIdx.y, kv_head = blockIdx.x, batch = blockIdx.z;
  const int kv0 = jt * BN;
  const int rep = p.Hq / p.Hkv;
  const int n_qt = (p.S + BM - 1) / BM;
  const int i_lo = p.causal ? (kv0 / BM) : 0;
  int i_hi = n_qt;
  if (p.window > 0) i_hi = min(n_qt, (kv0 + BN - 1 + p.window - 1) / BM + 1);
  const int per_head = max(i_hi - i_lo, 0);
  const int n_iters = per_head * rep;
  WaitCtx wctx{abort_flag, p.status};

  const int cta_lin = int(blockIdx.x) + int(gridDim.x) * (int(blockIdx.y) + int(gridDim.y) * int(blockIdx.z));
  unsigned long long* tr_buf = nullptr;
  int tr_n = 0;
  if (TRACE && trace != nullptr && cta_lin < trace_ctas && lane == 0)
    tr_buf = trace + (size_t(cta_lin) * BWD2_WARPS + warp) * BWD2_TRACE_EV;
  auto tr = [&](int code) {
    if (TRACE) {
      if (tr_buf != nullptr && tr_n < BWD2_TRACE_EV)
        tr_buf[tr_n++] = (static_cast<unsigned long long>(clock64()) << 8) | static_cast<unsigned long long>(code);
    }
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    for (int i = 0; i < QS; ++i) {
      mbar_init(&qdo_full[i], 1);
      mbar_init(&qdo_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
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
      if (n_iters > 0) {   // nobody waits for K / V otherwise, and a copy must not outlive the CTA
        mbar_expect_tx(kv_full, 2 * Cfg::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_4d(sK + b * BLK, &tmap_k, kv_full, b * 64, kv_head, kv0, batch);
          tma_load_4d(sV + b * BLK, &tmap_v, kv_full, b * 64, kv_head, kv0, batch);
        }
      }
      for (int it = 0; it < n_iters; ++it) {
        const int st = it % QS;
        const uint32_t ph = uint32_t(it / QS) & 1;
        const int head = kv_head * rep + it / per_head;
        const int q0 = (i_lo + it % per_head) * BM;
        if (!zb_in_bounds(q0 >= 0 && q0 < p.S && head < p.Hq && kv0 < p.S, p.status, 8)) break;
        if (!mbar_wait(&qdo_empty[st], ph ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
        tr(TB_TMA_STAGE_FREE);
        mbar_expect_tx(&qdo_full[st], 2 * Cfg::TILE_BYTES + (DQ ? 0 : 1024));
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_4d(sQ + st * Cfg::TILE_BYTES + b * BLK, &tmap_q, &qdo_full[st], b * 64, head, q0, batch);
          tma_load_4d(sDO + st * Cfg::TILE_BYTES + b * BLK, &tmap_do, &qdo_full[st], b * 64, head, q0, batch);
        }
        if constexpr (!DQ) {
          // lse (log2 units) and delta of the tile's 128 queries: 512 bytes each, next to the stage they belong to
          // (rows of the statistics buffer are padded to a multiple of 128 entries, q0 is a multiple of 128)
          const float* row = stats + (size_t(batch) * p.Hq + head) * 2 * size_t(s_pad) + q0;
          bulk_load_1d(sDS + st * 1024, row, 512, &qdo_full[st]);
          bulk_load_1d(sDS + st * 1024 + 512, row + s_pad, 512, &qdo_full[st]);
        }
        tr(TB_TMA_ISSUED);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_iters > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, false, false);  // K-major A and B
      constexpr uint32_t idesc_dkv = umma_idesc_bf16(128, D, false, true);   // A from TMEM, B = [q rows][d] (N-major)
      // D = 128: A = K (M = head dim, M-major), B = dS^T tile (N = queries, N-major); D = 64: A = dS^T tile, B = K
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, D == 128 ? 128 : D, true, true);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), ds_addr = smem_u32(sDS);
      const uint32_t r_s = tmem_base, r_dp = tmem_base + Cfg::DP_COL;
      bool ok = mbar_wait(kv_full, 0, wctx, ST_TIMEOUT_FULL);
      auto issue_a = [&](uint32_t q_addr) {  // S^T = K Q^T
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
          umma_f16_ss(r_s, umma_desc_kmajor(k_addr + off), umma_desc_kmajor(q_addr + off), idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
      };
      auto issue_b = [&](uint32_t do_addr) {  // dP^T = V dO^T
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
          umma_f16_ss(r_dp, umma_desc_kmajor(v_addr + off), umma_desc_kmajor(do_addr + off), idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(dp_full);
      };
      if (ok) ok = mbar_wait(&qdo_full[0], 0, wctx, ST_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_a(smem_u32(sQ));
        issue_b(smem_u32(sDO));
        tr(TB_MMA_B_ISSUED);
      }
      for (int it = 0; it < n_iters && ok; ++it) {
        const int st = it % QS;
        const uint32_t q_addr = smem_u32(sQ + st * Cfg::TILE_BYTES), do_addr = smem_u32(sDO + st * Cfg::TILE_BYTES);
        if (!mbar_wait(pds_full, uint32_t(it) & 1, wctx, ST_TIMEOUT_MISC)) break;
        tr(TB_MMA_PDS_READY);
        tc_fence_after();
        // D: dV += P^T dO, E: dK += dS^T Q  (reduction over the 128 queries; bf16 A operands sit in the
        // first 32 columns of each 64-column half of R_S / R_dP)
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {
          const uint32_t acol = uint32_t(kk / 4) * 64 + uint32_t(kk % 4) * 8;
          umma_f16_ts(tmem_base + Cfg::DV_COL, r_s + acol, umma_desc_mnmajor(do_addr + kk * 2048, BLK), idesc_dkv,
                      (it | kk) != 0 ? 1u : 0u);
        }
        if constexpr (!DQ) {
          // S^T of the next step right behind D (which was P^T's last reader), ahead of E: the next step's
          // exponentials then start 8 products earlier, while E and B are still running
          if (it + 1 < n_iters) {
            const int sn = (it + 1) % QS;
            if (!mbar_wait(&qdo_full[sn], uint32_t((it + 1) / QS) & 1, wctx, ST_TIMEOUT_FULL)) break;
            tr(TB_MMA_QDO_READY);
            tc_fence_after();
            issue_a(smem_u32(sQ + sn * Cfg::TILE_BYTES));
            tr(TB_MMA_A_ISSUED);
          }
        }
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {
          const uint32_t acol = uint32_t(kk / 4) * 64 + uint32_t(kk % 4) * 8;
          umma_f16_ts(tmem_base + Cfg::DK_COL, r_dp + acol, umma_desc_mnmajor(q_addr + kk * 2048, BLK), idesc_dkv,
                      (it | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&qdo_empty[st]);
        if constexpr (!DQ) {
          if (it + 1 == n_iters) umma_commit(dq_full);   // every dK / dV product is done: the write-out may start
          tr(TB_MMA_DEF_ISSUED);
          if (it + 1 < n_iters) {
            issue_b(smem_u32(sDO + ((it + 1) % QS) * Cfg::TILE_BYTES));   // overwrites R_dP behind E, its last reader
            tr(TB_MMA_B_ISSUED);
          }
          continue;
        }
        if constexpr (DQ) {
        // F: dQ = dS K  (reduction over the 128 keys) into R_dP, right behind E which read dS^T from it.
        // For D = 128 the product is formed transposed, dQ^T = K^T dS^T (same two shared-memory tiles with
        // the operand roles swapped): head-dim index on the TMEM lanes, so that the 32 lanes of a warp add
        // to 32 consecutive floats of one query row (one full 128-byte line per instruction) in G.
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          if constexpr (D == 128)
            umma_f16_ss(r_dp, umma_desc_mnmajor(k_addr + kk * 2048, BLK), umma_desc_mnmajor(ds_addr + kk * 2048, BLK),
                        idesc_dq, kk != 0 ? 1u : 0u);
          else
            umma_f16_ss(r_dp, umma_desc_mnmajor(ds_addr + kk * 2048, BLK), umma_desc_mnmajor(k_addr + kk * 2048, BLK),
                        idesc_dq, kk != 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
        }
        tr(TB_MMA_DEF_ISSUED);
        if (it + 1 < n_iters) {
          const int sn = (it + 1) % QS;
          if (!mbar_wait(&qdo_full[sn], uint32_t((it + 1) / QS) & 1, wctx, ST_TIMEOUT_FULL)) break;
          tr(TB_MMA_QDO_READY);
          tc_fence_after();
          issue_a(smem_u32(sQ + sn * Cfg::TILE_BYTES));
          tr(TB_MMA_A_ISSUED);
          if constexpr (DQ) {
            // dQ_it sits in R_dP until the compute warps have drained it
            if (!mbar_wait(dq_empty, uint32_t(it) & 1, wctx, ST_TIMEOUT_TMEM_EMPTY)) break;
            tr(TB_MMA_DQ_EMPTY);
            tc_fence_after();
          }
          issue_b(smem_u32(sDO + sn * Cfg::TILE_BYTES));
          tr(TB_MMA_B_ISSUED);
        }
      }
    }
  } else {
    // ------------------------------ compute warps ------------------------------
    const int half = warp >> 2;                  // which 64 query columns of S^T / dP^T (C), which d half (G, final)
    const int t = (warp & 3) * 32 + lane;        // TMEM lane: key row (C, final write), query row (G)
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const int key = kv0 + t;
    const bool key_ok = key < p.S;
    uint8_t* ds_row = sDS + half * BLK + t * 128;  // this thread's 128-byte row of its 64-query block
    bool ok = true;
    for (int it = 0; it < n_iters; ++it) {
      const int head = kv_head * rep + it / per_head;
      const int q0 = (i_lo + it % per_head) * BM;
      const int qc0 = q0 + half * 64;            // first query column of this thread
      // statistics of the tile's queries: global rows indexed by the absolute query (one-kernel form), or the
      // copy the producer placed in shared memory with the stage, indexed from the tile's first query
      const float* lse_q = stats + (size_t(batch) * p.Hq + head) * 2 * size_t(s_pad);
      const float* delta_q = lse_q + s_pad;
      if constexpr (!DQ) {
        const int st = it % QS;
        if (!__all_sync(0xffffffffu, mbar_wait(&qdo_full[st], uint32_t(it / QS) & 1, wctx, ST_TIMEOUT_FULL))) { ok = false; break; }
        lse_q = reinterpret_cast<const float*>(sDS + st * 1024) - q0;
        delta_q = reinterpret_cast<const float*>(sDS + st * 1024 + 512) - q0;
      }
      const bool need_mask = (p.causal && kv0 + BN - 1 > q0) || (p.window > 0 && kv0 < q0 + BM - p.window) ||
                             (kv0 + BN > p.S) || (q0 + BM > p.S);
      // ---- C1: P^T = exp2(S^T c - lse_q), kept as packed bf16 pairs (queries 2i, 2i+1) ----
      if (!__all_sync(0xffffffffu, mbar_wait(s_full, uint32_t(it) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tr(TB_S_READY);
      tc_fence_after();
      // lse_q (already in log2 units) and delta_q are the same for every lane: 16-byte loads from the
      // padded statistics rows
      auto load4 = [&](const float* base, int q, float (&v)[4]) {
        const float4 a = DQ ? __ldg(reinterpret_cast<const float4*>(base + q)) : *reinterpret_cast<const float4*>(base + q);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
      };
      uint32_t pp[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rs[32];
        tmem_ld32(lane_addr + uint32_t(half * 64 + c * 32), rs);
        tmem_wait_ld();
#pragma unroll
        // the mask test is hoisted out of the element loop: one branch per chunk, not one per element
        if (need_mask) {
#pragma unroll
          for (int k = 0; k < 32; k += 4) {
            float l4[4], e[4];
            load4(lse_q, qc0 + c * 32 + k, l4);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int q = qc0 + c * 32 + k + u;
              const float pe = exp2f(fmaf(__uint_as_float(rs[k + u]), p.scale_log2, -l4[u]));
              const bool vis = key_ok && (q < p.S) && (!p.causal || key <= q) && (p.window <= 0 || q - key < p.window);
              e[u] = vis ? pe : 0.f;
            }
            pp[c * 16 + (k >> 1)] = pack_bf16x2(e[0], e[1]);
            pp[c * 16 + (k >> 1) + 1] = pack_bf16x2(e[2], e[3]);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 32; k += 4) {
            float l4[4], e[4];
            load4(lse_q, qc0 + c * 32 + k, l4);
#pragma unroll
            for (int u = 0; u < 4; ++u) e[u] = exp2f(fmaf(__uint_as_float(rs[k + u]), p.scale_log2, -l4[u]));
            pp[c * 16 + (k >> 1)] = pack_bf16x2(e[0], e[1]);
            pp[c * 16 + (k >> 1) + 1] = pack_bf16x2(e[2], e[3]);
          }
        }
      }
      {
        uint32_t lo16[16], hi16[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) { lo16[k] = pp[k]; hi16[k] = pp[16 + k]; }
        tmem_st16(lane_addr + uint32_t(half * 64), lo16);
        tmem_st16(lane_addr + uint32_t(half * 64 + 16), hi16);
      }
      tr(TB_P_DONE);
      // ---- C2: dS^T = P^T (dP^T - delta_q) scale -> TMEM (bf16 over R_dP) and shared memory ----
      if (!__all_sync(0xffffffffu, mbar_wait(dp_full, uint32_t(it) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tr(TB_DP_READY);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rd[32];
        tmem_ld32(lane_addr + uint32_t(Cfg::DP_COL + half * 64 + c * 32), rd);
        tmem_wait_ld();
        uint32_t ds[16];
#pragma unroll
        for (int k = 0; k < 32; k += 4) {
          float d4[4];
          load4(delta_q, qc0 + c * 32 + k, d4);
          const float2 pa = unpack_bf16x2(pp[c * 16 + (k >> 1)]), pb = unpack_bf16x2(pp[c * 16 + (k >> 1) + 1]);
          const float s0 = pa.x * (__uint_as_float(rd[k]) - d4[0]) * p.scale;
          const float s1 = pa.y * (__uint_as_float(rd[k + 1]) - d4[1]) * p.scale;
          const float s2 = pb.x * (__uint_as_float(rd[k + 2]) - d4[2]) * p.scale;
          const float s3 = pb.y * (__uint_as_float(rd[k + 3]) - d4[3]) * p.scale;
          ds[k >> 1] = pack_bf16x2(s0, s1);
          ds[(k >> 1) + 1] = pack_bf16x2(s2, s3);
        }
        // the other half's threads read columns [64 h', 64 h' + 64) only, so writing the packed
        // values over this half's own first 32 columns cannot disturb them
        tmem_st16(lane_addr + uint32_t(Cfg::DP_COL + half * 64 + c * 16), ds);
        if constexpr (DQ) {
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const int ch = c * 4 + v4;  // 16-byte chunk (8 queries) within the 128-byte row
          uint4 u = make_uint4(ds[v4 * 4 + 0], ds[v4 * 4 + 1], ds[v4 * 4 + 2], ds[v4 * 4 + 3]);
          *reinterpret_cast<uint4*>(ds_row + ((ch ^ (t & 7)) << 4)) = u;
        }
        }
      }
      tmem_wait_st();
      if constexpr (DQ) fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      tr(TB_DS_DONE);
      if constexpr (DQ) {
      // ---- G: dQ tile (lanes = query rows now) -> global fp32 accumulator ----
      if (!__all_sync(0xffffffffu, mbar_wait(dq_full, uint32_t(it) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tr(TB_DQ_READY);
      tc_fence_after();
      if constexpr (D == 128) {
        // lanes = head-dim index t, columns = queries: this thread adds element t of 64 query rows
        const size_t row_stride = size_t(p.Hq) * D;
        float* dq_col = p.dq_acc + (size_t(batch) * p.S + q0) * row_stride + size_t(head) * D + t;
#pragma unroll 1
        for (int c = half * 2; c < half * 2 + 2; ++c) {
          uint32_t r[32];
          tmem_ld32(lane_addr + uint32_t(Cfg::DP_COL + c * 32), r);
          tmem_wait_ld();
          const int nq = min(32, p.S - (q0 + c * 32));   // query rows of this chunk that exist (warp-uniform)
#pragma unroll
          for (int k = 0; k < 32; ++k)
            if (k < nq) red_add_f32(dq_col + size_t(c * 32 + k) * row_stride, __uint_as_float(r[k]));
        }
      } else {
      const int qrow = q0 + t;
      float* dq_row = p.dq_acc + (size_t(batch) * p.S + qrow) * (size_t(p.Hq) * D) + size_t(head) * D;
#pragma unroll 1
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t r[32];
        tmem_ld32(lane_addr + uint32_t(Cfg::DP_COL + c * 32), r);
        tmem_wait_ld();
        if (qrow < p.S) {
#pragma unroll
          for (int v4 = 0; v4 < 8; ++v4)
            red_add_v4_f32(dq_row + c * 32 + v4 * 4, __uint_as_float(r[v4 * 4 + 0]), __uint_as_float(r[v4 * 4 + 1]),
                           __uint_as_float(r[v4 * 4 + 2]), __uint_as_float(r[v4 * 4 + 3]));
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);
      tr(TB_DQ_DRAINED);
      }
    }
    if constexpr (!DQ) {
      // the single dq_full arrival follows the last dK / dV product
      if (ok && n_iters > 0) ok = mbar_wait(dq_full, 0, wctx, ST_TIMEOUT_TMEM_FULL);
      tc_fence_after();
    }
    // ------------------------------ dK / dV write-out ------------------------------
    // the last dq_full arrival also covers every dK / dV MMA issued before it
    const int width = (p.Hq + 2 * p.Hkv) * D;
    ok = __all_sync(0xffffffffu, ok);
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const uint32_t col0 = which == 0 ? Cfg::DK_COL : Cfg::DV_COL;
      __nv_bfloat16* dst = p.dqkv + (size_t(batch) * p.S + key) * width +
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
        if (ok && key_ok) {
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

// stats[(b, h)][0][s] = lse * log2(e), stats[(b, h)][1][s] = sum_d dO * O; rows padded to s_pad
// entries that this kernel never writes (they must have been zeroed once). One warp per (token, head).
__global__ void attn_bwd2_stats_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                       const float* __restrict__ lse, float* __restrict__ stats, int B, int S, int Hq,
                                       int D, int s_pad) {
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
    float* row = stats + (b * Hq + h) * 2 * long(s_pad);
    row[s] = lse[(b * Hq + h) * S + s] * 1.4426950408889634f;
    row[s_pad + s] = acc;
  }
}

static int make_head_tmap_bwd2(CUtensorMap* out, const __nv_bfloat16* base, int B, int S, int heads, int D, int width) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(heads), uint64_t(S), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(width) * 2, uint64_t(width) * 2 * uint64_t(S)};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_nd_bf16(out, base, 4, dims, strides, box);
}

template <int D, bool TRACE, bool DQ = true>
static int launch_bwd2(const __nv_bfloat16* qkv, const __nv_bfloat16* d_o, const AttnBwdParams& p, const float* stats,
                       int s_pad, unsigned long long* trace, int trace_ctas, cudaStream_t stream) {
  using Cfg = AttnBwd2Cfg<D>;
  const int width = (p.Hq + 2 * p.Hkv) * D;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_head_tmap_bwd2(&tq, qkv, p.B, p.S, p.Hq, D, width))) return rc;
  if ((rc = make_head_tmap_bwd2(&tk, qkv + size_t(p.Hq) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  if ((rc = make_head_tmap_bwd2(&tv, qkv + size_t(p.Hq + p.Hkv) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  if ((rc = make_head_tmap_bwd2(&tdo, d_o, p.B, p.S, p.Hq, D, p.Hq * D))) return rc;
  auto kern = flash_bwd2_kernel<D, TRACE, DQ>;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set = true;
  }
  dim3 grid(p.Hkv, (p.S + 127) / 128, p.B);
  kern<<<grid, 32 * BWD2_WARPS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tdo, p, stats, s_pad, trace, trace_ctas);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

int attn_bwd_dq(const __nv_bfloat16* qkv, const __nv_bfloat16* d_o, const AttnBwdParams& p, const float* stats, int s_pad,
                int D, cudaStream_t stream);   // flash_bwd_dq.cu

}  // namespace zb

extern "C" {

int zb_flash_bwd2_trace_events() { return zb::BWD2_TRACE_EV; }
int zb_flash_bwd2_trace_warps() { return zb::BWD2_WARPS; }

int zb_flash_bwd2_stats_floats(int B, int S, int Hq) { return B * Hq * 2 * ((S + 127) / 128 * 128); }

// Scratch: stats fp32 [zb_flash_bwd2_stats_floats(B, S, Hq)], zeroed once by the caller (rows are padded to a
// multiple of 128 and the padding is never written); dq_acc fp32 [B*S*Hq*D], zero on entry (left zero).
// trace: nullptr, or a zeroed device buffer of trace_ctas * warps * events 64-bit words.
int zb_flash_bwd2(const void* d_o, const void* qkv, const void* o, const float* lse, void* dqkv, float* stats,
                  float* dq_acc, int B, int S, int Hq, int Hkv, int D, int causal, int window, float softmax_scale,
                  int* status, unsigned long long* trace, int trace_ctas, cudaStream_t stream) {
  using namespace zb;
  if (B <= 0 || S <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) ZB_FAIL(-1, "attention: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  if (D != 64 && D != 128) ZB_FAIL(-1, "attention: head dim %d unsupported (64 or 128)", D);
  auto DO = static_cast<const __nv_bfloat16*>(d_o);
  auto O = static_cast<const __nv_bfloat16*>(o);
  auto QKV = static_cast<const __nv_bfloat16*>(qkv);
  const int s_pad = (S + 127) / 128 * 128;
  {
    const long warps = long(B) * S * Hq;
    const long blocks = (warps * 32 + 255) / 256;
    attn_bwd2_stats_kernel<<<(unsigned)blocks, 256, 0, stream>>>(O, DO, lse, stats, B, S, Hq, D, s_pad);
    ZB_CUDA_OK(cudaGetLastError());
  }
  AttnBwdParams p;
  p.lse = lse; p.delta = nullptr; p.dq_acc = dq_acc;
  p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.window = window; p.causal = causal;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  const bool trc = trace != nullptr && trace_ctas > 0;
  int rc;
  if (D == 128) rc = trc ? launch_bwd2<128, true>(QKV, DO, p, stats, s_pad, trace, trace_ctas, stream)
                         : launch_bwd2<128, false>(QKV, DO, p, stats, s_pad, nullptr, 0, stream);
  else rc = trc ? launch_bwd2<64, true>(QKV, DO, p, stats, s_pad, trace, trace_ctas, stream)
                : launch_bwd2<64, false>(QKV, DO, p, stats, s_pad, nullptr, 0, stream);
  if (rc) return rc;
  return attn_bwd_finish_dq(dq_acc, p.dqkv, B, S, Hq, Hkv, D, stream);
}

// Two-kernel backward without atomics: statistics pass, then dK / dV per key tile (this file's kernel without
// its dQ part) and dQ per query tile (flash_bwd_dq.cu); the two main kernels are independent of each other.
// Scratch: stats fp32 [zb_flash_bwd2_stats_floats(B, S, Hq)], zeroed once by the caller.
int zb_flash_bwd3(const void* d_o, const void* qkv, const void* o, const float* lse, void* dqkv, float* stats,
                  int B, int S, int Hq, int Hkv, int D, int causal, int window, float softmax_scale, int* status,
                  int parts, unsigned long long* trace, int trace_ctas, cudaStream_t stream) {
  // parts: 3 = the whole backward; 1 = statistics + dK / dV kernel only, 2 = dQ kernel only (needs the
  // statistics of an earlier call) - for timing the two halves separately
  using namespace zb;
  if (B <= 0 || S <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) ZB_FAIL(-1, "attention: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  if (D != 64 && D != 128) ZB_FAIL(-1, "attention: head dim %d unsupported (64 or 128)", D);
  auto DO = static_cast<const __nv_bfloat16*>(d_o);
  auto O = static_cast<const __nv_bfloat16*>(o);
  auto QKV = static_cast<const __nv_bfloat16*>(qkv);
  const int s_pad = (S + 127) / 128 * 128;
  if (parts & 1) {
    const long warps = long(B) * S * Hq;
    const long blocks = (warps * 32 + 255) / 256;
    attn_bwd2_stats_kernel<<<(unsigned)blocks, 256, 0, stream>>>(O, DO, lse, stats, B, S, Hq, D, s_pad);
    ZB_CUDA_OK(cudaGetLastError());
  }
  AttnBwdParams p;
  p.lse = lse; p.delta = nullptr; p.dq_acc = nullptr;
  p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.window = window; p.causal = causal;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  int rc = 0;
  const bool trc = trace != nullptr && trace_ctas > 0;     // phase trace of the dK / dV kernel (as in zb_flash_bwd2)
  if (parts & 1) {
    if (D == 128) rc = trc ? launch_bwd2<128, true, false>(QKV, DO, p, stats, s_pad, trace, trace_ctas, stream)
                           : launch_bwd2<128, false, false>(QKV, DO, p, stats, s_pad, nullptr, 0, stream);
    else rc = trc ? launch_bwd2<64, true, false>(QKV, DO, p, stats, s_pad, trace, trace_ctas, stream)
                  : launch_bwd2<64, false, false>(QKV, DO, p, stats, s_pad, nullptr, 0, stream);
  }
  if (rc) return rc;
  return (parts & 2) ? attn_bwd_dq(QKV, DO, p, stats, s_pad, D, stream) : 0;
}

}  // extern "C"
