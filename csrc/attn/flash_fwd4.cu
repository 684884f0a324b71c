// Flash attention forward, two query tiles per CTA, one MMA issuer, score rows held in
// registers (sm_100a).  Same interface and memory layouts as flash_fwd.cu.
//
// Per CTA: 256 query rows of one head = two chains (c = 0: rows [q0, q0+128), c = 1: the next
// 128), K/V tiles of 128 keys streamed through one ring of shared-memory slots
// (K_j, V_j, K_j+1, V_j+1, ...).  Per chain and key tile j:
//     S_c = Q_c K_j^T         tcgen05.mma, SS form, fp32 in TMEM (128 columns)
//     P_c = exp2(S c - m c)   the chain's 128 softmax threads, one row each: the whole row
//                             (128 fp32) is read from TMEM ONCE and stays in registers for the
//                             maximum, the exponentials and the row sum; P goes back as packed
//                             bf16 over columns [0, 64) of S_c in two halves, each announced
//                             on its own barrier so P V can start on the first 64 keys
//     O_c += P_c V_j          tcgen05.mma, TS form (A = P from tensor memory)
// ONE thread issues every MMA of both chains in the order
//     PV_0(j) QK_0(j+1) PV_1(j) QK_1(j+1) ...
// and never waits for an MMA to finish: the tensor pipe executes in issue order, so QK_c(j+1)
// may overwrite S_c/P_c right behind PV_c(j), and while chain 0 is in its softmax the pipe
// runs chain 1's pair.  The issuer only waits for data (ring slots, P halves).
// O is rescaled in TMEM only when a row maximum grew by more than 2^8 (final normalisation
// absorbs the slack).
//
// Warps 0-3: softmax chain 0, 4-7: softmax chain 1, 8: MMA issuer + TMEM owner, 9: TMA producer,
// 10-11: idle.  The third warpgroup gives registers back (setmaxnreg.dec) so that the softmax
// warpgroups can hold a 128-value score row each (setmaxnreg.inc).
// TMEM: S_0 [0,128) S_1 [128,256) O_0 [256,256+D) O_1 [384,384+D).
//
// With TRACE the first `trace_ctas` CTAs record (clock64, code) pairs per warp at phase
// boundaries into a global buffer; zorse_b200/profiler/attn_trace.py turns them into a
// per-phase timeline.
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

struct AttnFwd4Params {
  __nv_bfloat16* O;
  float* lse;
  int B, S, Hq, Hkv;
  int window, causal;
  float scale_log2;
  int ldo;
  int* status;
  unsigned long long* trace;  // [trace_ctas][10 warps][TRACE_EV] or nullptr
  int trace_ctas;
};

constexpr int FWD4_TRACE_EV = 256;
constexpr int FWD4_WARPS = 12;
// setmaxnreg moves registers inside what the CTA was given at launch: 384 threads x 168 registers
// (the launch bound) = 64512.  The three warpgroups must add up to exactly that, or the second
// `inc` waits for registers that never come: 2 * 128 * 208 + 128 * 88 = 64512.
constexpr int FWD4_SOFTMAX_REGS = 208;
constexpr int FWD4_OTHER_REGS = 88;
static_assert(2 * 128 * FWD4_SOFTMAX_REGS + 128 * FWD4_OTHER_REGS == 384 * 168, "register budget of the three warpgroups");

template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

template <int D>
struct AttnFwd4Cfg {
  static constexpr int BM = 128, BN = 128;
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int NSLOT = (D == 128) ? 5 : 8;
  static constexpr int SMEM_BYTES = (2 + NSLOT) * TILE_BYTES + 1024 + 512;
  static constexpr int THREADS = 32 * FWD4_WARPS;
};

// trace codes (low byte of an event; bits 8.. = clock64)
enum : int {
  TR_S_READY = 1, TR_S_LOADED = 2, TR_MAX_DONE = 3, TR_P_HALF0 = 4, TR_P_HALF1 = 5, TR_EPI_BEGIN = 6, TR_EPI_END = 7,
  TR_MMA_V_READY = 16, TR_MMA_P0_READY = 17, TR_MMA_P1_READY = 18, TR_MMA_PV_ISSUED = 19, TR_MMA_K_READY = 20,
  TR_MMA_QK_ISSUED = 21,
  TR_TMA_SLOT_FREE = 32, TR_TMA_ISSUED = 33,
};

template <int D, bool TRACE, int MODE>
__global__ void __launch_bounds__(32 * FWD4_WARPS, 1)
flash_fwd4_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const AttnFwd4Params p) {
  using Cfg = AttnFwd4Cfg<D>;
  constexpr int BM = 128, BN = 128, NSLOT = Cfg::NSLOT, DB = D / 64, BLK = 128 * 128;
  constexpr bool PACKED = MODE >= 1;   // two-wide fp32 fma / add, three-input maximum
  constexpr bool POLY = MODE >= 2;     // every fourth exponential on the fma pipe instead of MUFU
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                               // two tiles
  uint8_t* sR = sQ + 2 * Cfg::TILE_BYTES;           // ring of NSLOT tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sR + NSLOT * Cfg::TILE_BYTES);
  uint64_t* q_full = bars;                  // [2]
  uint64_t* r_full = bars + 2;              // [NSLOT]
  uint64_t* r_empty = r_full + NSLOT;       // [NSLOT]
  uint64_t* s_full = r_empty + NSLOT;       // [2]
  uint64_t* p_half = s_full + 2;            // [2 chains][2 halves], 4 arrivals each
  uint64_t* o_done = p_half + 4;            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_pairs = (p.S + 2 * BM - 1) / (2 * BM);
  // grid = (heads, query pairs, batch): CTAs are dispatched x-fastest, so every head's heaviest
  // (latest) pair starts first and the light ones fill the tail of the last wave
  const int pair = n_pairs - 1 - int(blockIdx.y);
  const int head = blockIdx.x, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int n_kv = (p.S + BN - 1) / BN;
  int lo[2], hi[2];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int q0 = (2 * pair + c) * BM;
    lo[c] = 0;
    hi[c] = n_kv;
    if (p.causal) hi[c] = min(hi[c], (q0 + BM - 1) / BN + 1);
    if (p.window > 0) lo[c] = max(0, (q0 - p.window + 1) / BN);
    if (q0 >= p.S) { lo[c] = 0; hi[c] = 0; }
  }
  const bool act0 = hi[0] > lo[0], act1 = hi[1] > lo[1];
  const int j_lo = act1 ? (act0 ? min(lo[0], lo[1]) : lo[1]) : lo[0];
  const int j_hi = max(hi[0], hi[1]);
  const int n_tiles = max(j_hi - j_lo, 0);
  WaitCtx wctx{abort_flag, p.status};

  // ---- trace ----
  const int cta_lin = int(blockIdx.x) + int(gridDim.x) * (int(blockIdx.y) + int(gridDim.y) * int(blockIdx.z));
  unsigned long long* tr_buf = nullptr;
  int tr_n = 0;
  if (TRACE && p.trace != nullptr && cta_lin < p.trace_ctas && lane == 0)
    tr_buf = p.trace + (size_t(cta_lin) * FWD4_WARPS + warp) * FWD4_TRACE_EV;
  auto tr = [&](int code) {
    if (TRACE) {
      if (tr_buf != nullptr && tr_n < FWD4_TRACE_EV)
        tr_buf[tr_n++] = (static_cast<unsigned long long>(clock64()) << 8) | static_cast<unsigned long long>(code);
    }
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int c = 0; c < 2; ++c) {
      mbar_init(&q_full[c], 1);
      mbar_init(&s_full[c], 1);
      mbar_init(&p_half[2 * c], 4);
      mbar_init(&p_half[2 * c + 1], 4);
      mbar_init(&o_done[c], 1);
    }
    for (int i = 0; i < NSLOT; ++i) {
      mbar_init(&r_full[i], 1);
      mbar_init(&r_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    setmaxnreg_dec<FWD4_OTHER_REGS>();
    if (warp == 9) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (hi[c] <= lo[c]) continue;
          mbar_expect_tx(&q_full[c], Cfg::TILE_BYTES);
#pragma unroll
          for (int b = 0; b < DB; ++b)
            tma_load_4d(sQ + c * Cfg::TILE_BYTES + b * BLK, &tmap_q, &q_full[c], b * 64, head, (2 * pair + c) * BM, batch);
        }
        // ring entries: t = 2 i -> K of key tile j_lo + i, t = 2 i + 1 -> V of the same tile
        for (int t = 0; t < 2 * n_tiles; ++t) {
          const int slot = t % NSLOT;
          const uint32_t ph = uint32_t(t / NSLOT) & 1;
          const int kv0 = (j_lo + (t >> 1)) * BN;
          if (!zb_in_bounds(kv0 >= 0 && kv0 < p.S && kv_head < p.Hkv && batch < p.B, p.status, 8)) break;
          if (!mbar_wait(&r_empty[slot], ph ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
          tr(TR_TMA_SLOT_FREE);
          mbar_expect_tx(&r_full[slot], Cfg::TILE_BYTES);
          const CUtensorMap* tm = (t & 1) ? &tmap_v : &tmap_k;
#pragma unroll
          for (int b = 0; b < DB; ++b)
            tma_load_4d(sR + slot * Cfg::TILE_BYTES + b * BLK, tm, &r_full[slot], b * 64, kv_head, kv0, batch);
          tr(TR_TMA_ISSUED);
        }
      }
    } else if (warp == 8) {
      // ------------------------------ MMA issuer (both chains) ------------------------------
      if (lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16(BM, BN, false, false);
        constexpr uint32_t idesc_o = umma_idesc_bf16(BM, D, false, true);
        bool ok = true;
        int used[2] = {0, 0};  // tiles whose S has been issued, per chain
        int pv_done[2] = {0, 0};  // tiles whose P V has been issued, per chain
        auto chain_has = [&](int c, int j) { return hi[c] > lo[c] && j >= lo[c] && j < hi[c]; };
        auto issue_qk = [&](int c, int slot) -> bool {
          if (used[c] == 0) {
            if (!mbar_wait(&q_full[c], 0, wctx, ST_TIMEOUT_FULL)) return false;
            tc_fence_after();
          }
          const uint32_t q_addr = smem_u32(sQ + c * Cfg::TILE_BYTES), k_addr = smem_u32(sR + slot * Cfg::TILE_BYTES);
          const uint32_t s_col = tmem_base + uint32_t(c * 128);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
            umma_f16_ss(s_col, umma_desc_kmajor(q_addr + off), umma_desc_kmajor(k_addr + off), idesc_s, kk != 0 ? 1u : 0u);
          }
          umma_commit(&s_full[c]);
          ++used[c];
          return true;
        };
        // prologue: S_c = Q_c K_{j_lo}^T for the chains that use the first tile
        if (n_tiles > 0) {
          ok = mbar_wait(&r_full[0], 0, wctx, ST_TIMEOUT_FULL);
          tr(TR_MMA_K_READY);
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 2; ++c)
            if (ok && chain_has(c, j_lo)) ok = issue_qk(c, 0);
          if (ok) umma_commit(&r_empty[0]);
          tr(TR_MMA_QK_ISSUED);
        }
        for (int i = 0; i < n_tiles && ok; ++i) {
          const int j = j_lo + i;
          const int tv = 2 * i + 1, tk = 2 * i + 2;  // ring entries of V_j and K_{j+1}
          const int vslot = tv % NSLOT, kslot = tk % NSLOT;
          const bool more = i + 1 < n_tiles;
          if (!mbar_wait(&r_full[vslot], uint32_t(tv / NSLOT) & 1, wctx, ST_TIMEOUT_FULL)) { ok = false; break; }
          tr(TR_MMA_V_READY);
          bool k_ready = false;
          const uint32_t v_addr = smem_u32(sR + vslot * Cfg::TILE_BYTES);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (!ok) break;
            const uint32_t s_col = tmem_base + uint32_t(c * 128);
            const uint32_t o_col = tmem_base + uint32_t(256 + c * 128);
            if (chain_has(c, j)) {
              const uint32_t par = uint32_t(pv_done[c]) & 1;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                if (!mbar_wait(&p_half[2 * c + h], par, wctx, ST_TIMEOUT_MISC)) { ok = false; break; }
                tr(h == 0 ? TR_MMA_P0_READY : TR_MMA_P1_READY);
                tc_fence_after();
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                  const int kk = h * 4 + k4;
                  umma_f16_ts(o_col, s_col + uint32_t(kk * 8), umma_desc_mnmajor(v_addr + kk * 16 * 128, BLK), idesc_o,
                              (pv_done[c] | kk) != 0 ? 1u : 0u);
                }
              }
              if (!ok) break;
              ++pv_done[c];
              if (j == hi[c] - 1) umma_commit(&o_done[c]);
              tr(TR_MMA_PV_ISSUED);
            }
            if (more && chain_has(c, j + 1)) {
              if (!k_ready) {
                if (!mbar_wait(&r_full[kslot], uint32_t(tk / NSLOT) & 1, wctx, ST_TIMEOUT_FULL)) { ok = false; break; }
                tr(TR_MMA_K_READY);
                tc_fence_after();
                k_ready = true;
              }
              if (!issue_qk(c, kslot)) { ok = false; break; }
              tr(TR_MMA_QK_ISSUED);
            }
          }
          if (!ok) break;
          umma_commit(&r_empty[vslot]);
          if (more) {
            if (!k_ready) {
              // no chain uses K_{j+1} (cannot happen for a key tile inside the union, kept for safety)
              if (!mbar_wait(&r_full[kslot], uint32_t(tk / NSLOT) & 1, wctx, ST_TIMEOUT_FULL)) { ok = false; break; }
            }
            umma_commit(&r_empty[kslot]);
          }
        }
      }
    }
  } else {
    // ------------------------------ softmax warps of chain c ------------------------------
    setmaxnreg_inc<FWD4_SOFTMAX_REGS>();
    const int c = warp >> 2;
    const int t = threadIdx.x & 127;  // row inside the chain's query tile = TMEM lane
    const int q0 = (2 * pair + c) * BM;
    const int row = q0 + t;
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const uint32_t s_col = lane_addr + uint32_t(c * 128);
    const uint32_t o_col = lane_addr + uint32_t(256 + c * 128);
    const int my_lo = c ? lo[1] : lo[0];
    const int my_tiles = max((c ? hi[1] : hi[0]) - my_lo, 0);
    const float scale = p.scale_log2;
    float m_run = -INFINITY, l_run = 0.f;  // m_run in raw (unscaled) score units
    bool ok = true;
    for (int i = 0; i < my_tiles; ++i) {
      const int kv0 = (my_lo + i) * BN;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[c], uint32_t(i) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tr(TR_S_READY);
      tc_fence_after();
      // the whole score row: one TMEM round trip
      uint32_t s0[32], s1[32], s2[32], s3[32];
      tmem_ld32(s_col, s0);
      tmem_ld32(s_col + 32u, s1);
      tmem_ld32(s_col + 64u, s2);
      tmem_ld32(s_col + 96u, s3);
      tmem_wait_ld();
      tr(TR_S_LOADED);
      const bool need_mask = (p.causal && kv0 + BN - 1 > q0) || (p.window > 0 && kv0 < q0 + BM - p.window) ||
                             (kv0 + BN > p.S);
      if (need_mask) {
        auto mask32 = [&](uint32_t (&r)[32], int base) {
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const int col = kv0 + base + k;
            const bool vis = (col < p.S) && (!p.causal || col <= row) && (p.window <= 0 || row - col < p.window);
            r[k] = vis ? r[k] : 0xff800000u;  // -inf
          }
        };
        mask32(s0, 0);
        mask32(s1, 32);
        mask32(s2, 64);
        mask32(s3, 96);
      }
      float mx[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) mx[k] = -INFINITY;
      if (PACKED) {
        // three-input maximum: two new values per instruction, eight independent chains
#pragma unroll
        for (int k = 0; k < 32; k += 4) {
          mx[0] = fmax3(mx[0], __uint_as_float(s0[k]), __uint_as_float(s0[k + 1]));
          mx[1] = fmax3(mx[1], __uint_as_float(s0[k + 2]), __uint_as_float(s0[k + 3]));
          mx[2] = fmax3(mx[2], __uint_as_float(s1[k]), __uint_as_float(s1[k + 1]));
          mx[3] = fmax3(mx[3], __uint_as_float(s1[k + 2]), __uint_as_float(s1[k + 3]));
          mx[4] = fmax3(mx[4], __uint_as_float(s2[k]), __uint_as_float(s2[k + 1]));
          mx[5] = fmax3(mx[5], __uint_as_float(s2[k + 2]), __uint_as_float(s2[k + 3]));
          mx[6] = fmax3(mx[6], __uint_as_float(s3[k]), __uint_as_float(s3[k + 1]));
          mx[7] = fmax3(mx[7], __uint_as_float(s3[k + 2]), __uint_as_float(s3[k + 3]));
        }
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          mx[k & 1] = fmaxf(mx[k & 1], __uint_as_float(s0[k]));
          mx[2 + (k & 1)] = fmaxf(mx[2 + (k & 1)], __uint_as_float(s1[k]));
          mx[4 + (k & 1)] = fmaxf(mx[4 + (k & 1)], __uint_as_float(s2[k]));
          mx[6 + (k & 1)] = fmaxf(mx[6 + (k & 1)], __uint_as_float(s3[k]));
        }
      }
      const float tmax = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
      // running maximum; O is rescaled only when it grew by more than 8 in log2 units
      if (i == 0) {
        m_run = tmax;
      } else {
        const bool need = (tmax - m_run) * scale > 8.f;
        if (__any_sync(0xffffffffu, need)) {
          float alpha = 1.f;
          if (need) {
            alpha = (m_run == -INFINITY) ? 0.f : exp2f((m_run - tmax) * scale);
            m_run = tmax;
            l_run *= alpha;
          }
          // s_full(i) arrived => every MMA issued before it, including P V of tile i-1, is done
#pragma unroll 1
          for (int ch = 0; ch < D / 32; ++ch) {
            uint32_t r[32];
            tmem_ld32(o_col + uint32_t(ch * 32), r);
            tmem_wait_ld();
#pragma unroll
            for (int k = 0; k < 32; ++k) r[k] = __float_as_uint(__uint_as_float(r[k]) * alpha);
            tmem_st32(o_col + uint32_t(ch * 32), r);
          }
          tmem_wait_st();
        }
      }
      tr(TR_MAX_DONE);
      const float m_eff = (m_run == -INFINITY) ? 0.f : m_run;
      const float neg_mc = -m_eff * scale;
      float ls[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      auto exp_store = [&](uint32_t (&r)[32], uint32_t col_off) {
        uint32_t pk[16];
#pragma unroll
        for (int k = 0; k < 32; k += 2) {
          float x0, x1;
          if (PACKED) {
            ffma2(x0, x1, __uint_as_float(r[k]), __uint_as_float(r[k + 1]), scale, scale, neg_mc, neg_mc);
          } else {
            x0 = fmaf(__uint_as_float(r[k]), scale, neg_mc);
            x1 = fmaf(__uint_as_float(r[k + 1]), scale, neg_mc);
          }
          // with POLY keys 3, 7, 11, ... of the tile take the polynomial, the other three quarters MUFU
          const float e0 = exp2f(x0);
          const float e1 = (POLY && (k & 2)) ? exp2_poly3(x1) : exp2f(x1);
          const int a = ((k >> 1) & 3) * 2;
          if (PACKED) {
            fadd2(ls[a], ls[a + 1], ls[a], ls[a + 1], e0, e1);
          } else {
            ls[a] += e0;
            ls[a + 1] += e1;
          }
          pk[k >> 1] = pack_bf16x2(e0, e1);
        }
        tmem_st16(s_col + col_off, pk);
      };
      // keys [0, 64) -> P columns [0, 32); announce; keys [64, 128) -> columns [32, 64); announce
      exp_store(s0, 0u);
      exp_store(s1, 16u);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_half[2 * c]);
      tr(TR_P_HALF0);
      exp_store(s2, 32u);
      exp_store(s3, 48u);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_half[2 * c + 1]);
      tr(TR_P_HALF1);
      l_run += ((ls[0] + ls[1]) + (ls[2] + ls[3])) + ((ls[4] + ls[5]) + (ls[6] + ls[7]));
    }
    // ------------------------------ epilogue ------------------------------
    if (ok && my_tiles > 0) ok = mbar_wait(&o_done[c], 0, wctx, ST_TIMEOUT_MISC);
    ok = __all_sync(0xffffffffu, ok);
    tr(TR_EPI_BEGIN);
    tc_fence_after();
    const float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
    __nv_bfloat16* orow = p.O + (size_t(batch) * p.S + row) * p.ldo + head * D;
#pragma unroll 1
    for (int ch = 0; ch < D / 32; ++ch) {
      uint32_t r[32];
      if (my_tiles > 0) {
        tmem_ld32(o_col + uint32_t(ch * 32), r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) r[k] = 0u;
      }
      if (ok && row < p.S) {
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          uint4 u;
          u.x = pack_bf16x2(__uint_as_float(r[v4 * 8 + 0]) * inv_l, __uint_as_float(r[v4 * 8 + 1]) * inv_l);
          u.y = pack_bf16x2(__uint_as_float(r[v4 * 8 + 2]) * inv_l, __uint_as_float(r[v4 * 8 + 3]) * inv_l);
          u.z = pack_bf16x2(__uint_as_float(r[v4 * 8 + 4]) * inv_l, __uint_as_float(r[v4 * 8 + 5]) * inv_l);
          u.w = pack_bf16x2(__uint_as_float(r[v4 * 8 + 6]) * inv_l, __uint_as_float(r[v4 * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + ch * 32 + v4 * 8) = u;
        }
      }
    }
    if (ok && row < p.S && p.lse != nullptr) {
      const float m_eff = (m_run == -INFINITY) ? 0.f : m_run;
      p.lse[(size_t(batch) * p.Hq + head) * p.S + row] =
          (l_run > 0.f) ? (m_eff * scale + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
    tr(TR_EPI_END);
  }

  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static int make_head_tmap4(CUtensorMap* out, const __nv_bfloat16* base, int B, int S, int heads, int D, int width) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(heads), uint64_t(S), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(width) * 2, uint64_t(width) * 2 * uint64_t(S)};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_nd_bf16(out, base, 4, dims, strides, box);
}

template <int D, bool TRACE, int MODE>
static int launch_fwd4(const __nv_bfloat16* qkv, int width, const AttnFwd4Params& p, cudaStream_t stream) {
  using Cfg = AttnFwd4Cfg<D>;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_head_tmap4(&tq, qkv, p.B, p.S, p.Hq, D, width))) return rc;
  if ((rc = make_head_tmap4(&tk, qkv + size_t(p.Hq) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  if ((rc = make_head_tmap4(&tv, qkv + size_t(p.Hq + p.Hkv) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  auto kern = flash_fwd4_kernel<D, TRACE, MODE>;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set = true;
  }
  dim3 grid(p.Hq, (p.S + 255) / 256, p.B);
  kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace zb

extern "C" int zb_flash_fwd4_trace_events() { return zb::FWD4_TRACE_EV; }
extern "C" int zb_flash_fwd4_trace_warps() { return zb::FWD4_WARPS; }

// flags: 0 = scalar softmax math, 1 = two-wide fp32 fma / add and three-input maximum,
// 2 = as 1 and a quarter of the exponentials as a polynomial on the fma pipe.
// trace: nullptr, or a zeroed device buffer of trace_ctas * zb_flash_fwd4_trace_warps() * zb_flash_fwd4_trace_events() 64-bit words.
extern "C" int zb_flash_fwd4(const void* qkv, void* out, float* lse, int B, int S, int Hq, int Hkv, int D,
                             int causal, int window, float softmax_scale, int ldo, int* status, int flags,
                             unsigned long long* trace, int trace_ctas, cudaStream_t stream) {
  using namespace zb;
  if (B <= 0 || S <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) ZB_FAIL(-1, "attention: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  AttnFwd4Params p;
  p.O = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.window = window; p.causal = causal;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.ldo = ldo;
  p.status = status;
  p.trace = trace;
  p.trace_ctas = trace_ctas;
  const int width = (Hq + 2 * Hkv) * D;
  auto Q = static_cast<const __nv_bfloat16*>(qkv);
  const bool tr = trace != nullptr && trace_ctas > 0;
  const int mode = flags < 0 ? 0 : (flags > 2 ? 2 : flags);
#define ZB_FWD4_DISPATCH(DD)                                                                                  \
  do {                                                                                                        \
    if (tr) {                                                                                                 \
      if (mode == 0) return launch_fwd4<DD, true, 0>(Q, width, p, stream);                                    \
      if (mode == 1) return launch_fwd4<DD, true, 1>(Q, width, p, stream);                                    \
      return launch_fwd4<DD, true, 2>(Q, width, p, stream);                                                   \
    }                                                                                                         \
    if (mode == 0) return launch_fwd4<DD, false, 0>(Q, width, p, stream);                                     \
    if (mode == 1) return launch_fwd4<DD, false, 1>(Q, width, p, stream);                                     \
    return launch_fwd4<DD, false, 2>(Q, width, p, stream);                                                    \
  } while (0)
  if (D == 128) ZB_FWD4_DISPATCH(128);
  if (D == 64) ZB_FWD4_DISPATCH(64);
#undef ZB_FWD4_DISPATCH
  ZB_FAIL(-1, "attention: head dim %d unsupported (64 or 128)", D);
}
