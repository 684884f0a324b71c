// Flash attention forward, one 128-row query tile per CTA, EIGHT softmax warps (sm_100a).
//
// Same data flow as flash_fwd.cu (S double-buffered in TMEM, P staged through a swizzled
// shared tile, O in TMEM with lazy rescaling) but every query row is shared by two threads:
// warps 0-3 take key columns [0,64) of a tile, warps 4-7 columns [64,128).  Each scheduler
// then holds two softmax warps, so the MUFU pipe (exp2) and the FP32 pipe overlap and the
// softmax phase of a tile - the critical path of the kernel - takes about half as long.  The
// two halves of a row agree on the row maximum through shared memory and an mbarrier per
// pair of warps (bounded wait); row sums are kept per half and added at the end.
// Warp 8 = TMA producer, warp 9 = MMA issuer and TMEM owner.
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

struct AttnFwd3Params {
  __nv_bfloat16* O;
  float* lse;
  int B, S, Hq, Hkv;
  int window;  // 0 = unlimited; else key j visible to query i iff i - j < window
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  int ldo;           // row stride of O in elements
  int* status;
};

template <int D>
struct AttnFwd3Cfg {
  static constexpr int BM = 128, BN = 128;
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int K_BYTES = BN * D * 2;
  static constexpr int V_BYTES = BN * D * 2;
  static constexpr int P_BYTES = BM * BN * 2;
  static constexpr int KV_STAGES = 2;
  static constexpr int SMEM_BYTES = Q_BYTES + KV_STAGES * (K_BYTES + V_BYTES) + P_BYTES + 1024 + 256 + 3200;
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = 256;
};

__device__ __forceinline__ float fwd3_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(320, 1)
flash_fwd3_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const AttnFwd3Params p) {
  using Cfg = AttnFwd3Cfg<D>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, STAGES = Cfg::KV_STAGES;
  constexpr int DB = D / 64;  // 64-column blocks per head
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::Q_BYTES;
  uint8_t* sV = sK + STAGES * Cfg::K_BYTES;
  uint8_t* sP = sV + STAGES * Cfg::V_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + Cfg::P_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* k_full = bars + 1;             // STAGES
  uint64_t* k_empty = k_full + STAGES;     // STAGES
  uint64_t* v_full = k_empty + STAGES;     // STAGES
  uint64_t* v_empty = v_full + STAGES;     // STAGES
  uint64_t* s_full = v_empty + STAGES;     // 2
  uint64_t* s_empty = s_full + 2;          // 2
  uint64_t* p_full = s_empty + 2;          // 1
  uint64_t* pv_done = p_full + 1;          // 1
  uint64_t* xbar = pv_done + 1;            // 4: one per pair of warps sharing rows (2 arrivals)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xbar + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.S + BM - 1) / BM;
  const int qt = n_qt - 1 - int(blockIdx.x);  // heavy (late) tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qt * BM;
  int j_lo = 0, j_hi = (p.S + BN - 1) / BN;
  if (p.causal) j_hi = min(j_hi, (q0 + BM - 1) / BN + 1);
  if (p.window > 0) j_lo = max(0, (q0 - p.window + 1) / BN);
  const int n_tiles = j_hi - j_lo;
  WaitCtx wctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);
    }
    mbar_init(p_full, 8);
    mbar_init(pv_done, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&xbar[i], 2);
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
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int b = 0; b < DB; ++b) tma_load_4d(sQ + b * (BM * 128), &tmap_q, q_full, b * 64, head, q0, batch);
      for (int i = 0; i < n_tiles; ++i) {
        const int st = i % STAGES;
        const uint32_t ph = uint32_t(i / STAGES) & 1;
        const int kv0 = (j_lo + i) * BN;
        if (!mbar_wait(&k_empty[st], ph ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&k_full[st], Cfg::K_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          tma_load_4d(sK + st * Cfg::K_BYTES + b * (BN * 128), &tmap_k, &k_full[st], b * 64, kv_head, kv0, batch);
        if (!mbar_wait(&v_empty[st], ph ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&v_full[st], Cfg::V_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          tma_load_4d(sV + st * Cfg::V_BYTES + b * (BN * 128), &tmap_v, &v_full[st], b * 64, kv_head, kv0, batch);
      }
    }
  } else if (warp == 9) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BM, BN, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(BM, D, false, true);
      bool ok = mbar_wait(q_full, 0, wctx, ST_TIMEOUT_FULL);
      auto issue_s = [&](int i) -> bool {
        const int st = i % STAGES;
        const uint32_t ph = uint32_t(i / STAGES) & 1;
        const int sb = i & 1;
        if (!mbar_wait(&k_full[st], ph, wctx, ST_TIMEOUT_FULL)) return false;
        if (!mbar_wait(&s_empty[sb], (uint32_t(i >> 1) & 1) ^ 1, wctx, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK + st * Cfg::K_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = uint32_t(kk / 4) * (BM * 128) + uint32_t(kk % 4) * 32;
          umma_f16_ss(tmem_base + uint32_t(sb * BN), umma_desc_kmajor(q_addr + off),
                      umma_desc_kmajor(k_addr + off), idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[sb]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int i = 0; i < n_tiles && ok; ++i) {
        if (i + 1 < n_tiles) {
          ok = issue_s(i + 1);
          if (!ok) break;
        }
        const int st = i % STAGES;
        const uint32_t ph = uint32_t(i / STAGES) & 1;
        if (!mbar_wait(&v_full[st], ph, wctx, ST_TIMEOUT_FULL)) break;
        if (!mbar_wait(p_full, uint32_t(i) & 1, wctx, ST_TIMEOUT_MISC)) break;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP), v_addr = smem_u32(sV + st * Cfg::V_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint32_t aoff = uint32_t(kk / 4) * (BM * 128) + uint32_t(kk % 4) * 32;
          umma_f16_ss(tmem_base + Cfg::O_COL, umma_desc_kmajor(p_addr + aoff),
                      umma_desc_mnmajor(v_addr + kk * 16 * 128, BN * 128), idesc_o, (i | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(pv_done);
      }
    }
  } else {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int half = warp >> 2;                       // which 64 key columns of a tile
    const int qd = warp & 3;                          // TMEM lane quarter
    const int t = qd * 32 + lane;                     // query row within the tile = TMEM lane
    const int row = q0 + t;
    const uint32_t lane_addr = tmem_base + (uint32_t(qd * 32) << 16);
    float* xch = reinterpret_cast<float*>(const_cast<int*>(abort_flag) + 4);  // [2][128] exchange of half maxima / sums
    float m_run = -INFINITY, l_run = 0.f;             // l_run: this half's share of the row sum
    bool ok = true;
    uint32_t xphase = 0;
    for (int i = 0; i < n_tiles; ++i) {
      const int sb = i & 1;
      const int kv0 = (j_lo + i) * BN;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[sb], uint32_t(i >> 1) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tc_fence_after();
      float s[64];
      {
        uint32_t r0[32], r1[32];
        tmem_ld32(lane_addr + uint32_t(sb * BN + half * 64), r0);
        tmem_ld32(lane_addr + uint32_t(sb * BN + half * 64 + 32), r1);
        tmem_wait_ld();
#pragma unroll
        for (int k = 0; k < 32; ++k) { s[k] = __uint_as_float(r0[k]); s[32 + k] = __uint_as_float(r1[k]); }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);

      const bool need_mask = (p.causal && kv0 + BN - 1 > q0) || (p.window > 0 && kv0 < q0 + BM - p.window) ||
                             (kv0 + BN > p.S);
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int k = 0; k < 64; ++k) {
          const int col = kv0 + half * 64 + k;
          const bool vis = (col < p.S) && (!p.causal || col <= row) && (p.window <= 0 || row - col < p.window);
          s[k] = vis ? s[k] : -INFINITY;
          mx[k & 3] = fmaxf(mx[k & 3], s[k]);
        }
      } else {
#pragma unroll
        for (int k = 0; k < 64; ++k) mx[k & 3] = fmaxf(mx[k & 3], s[k]);
      }
      float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      // agree on the row maximum with the thread that holds the other 64 columns of this row
      xch[(i & 1) * 256 + half * 128 + t] = tmax;
      __syncwarp();
      if (lane == 0) mbar_arrive(&xbar[qd]);
      if (!__all_sync(0xffffffffu, mbar_wait(&xbar[qd], xphase, wctx, ST_TIMEOUT_MISC))) { ok = false; break; }
      xphase ^= 1;
      tmax = fmaxf(tmax, xch[(i & 1) * 256 + (half ^ 1) * 128 + t]);
      if (i == 0) {
        m_run = tmax;
      } else {
        // previous P V must have finished before P is overwritten or O is touched
        if (!__all_sync(0xffffffffu, mbar_wait(pv_done, uint32_t(i - 1) & 1, wctx, ST_TIMEOUT_MISC))) { ok = false; break; }
        tc_fence_after();
        const bool need = (tmax - m_run) * p.scale_log2 > 8.f;
        if (__any_sync(0xffffffffu, need)) {
          float alpha = 1.f;
          if (need) {
            alpha = (m_run == -INFINITY) ? 0.f : exp2f((m_run - tmax) * p.scale_log2);
            m_run = tmax;
            l_run *= alpha;
          }
#pragma unroll
          for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
            uint32_t r[32];
            tmem_ld32(lane_addr + uint32_t(Cfg::O_COL + c * 32), r);
            tmem_wait_ld();
#pragma unroll
            for (int k = 0; k < 32; ++k) r[k] = __float_as_uint(__uint_as_float(r[k]) * alpha);
            tmem_st32(lane_addr + uint32_t(Cfg::O_COL + c * 32), r);
          }
          tmem_wait_st();
        }
      }
      const float m_eff = (m_run == -INFINITY) ? 0.f : m_run;
      const float neg_mc = -m_eff * p.scale_log2;
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      // P -> shared memory, K-major 128-byte-swizzled: this half fills block `half` ([128 x 64])
      uint8_t* prow = sP + half * (BM * 128) + t * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float e[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          e[k] = exp2f(fmaf(s[c * 8 + k], p.scale_log2, neg_mc));   // masked entries are -inf -> 0
          ls[k & 3] += e[k];
        }
        uint4 u;
        u.x = pack_bf16x2(e[0], e[1]); u.y = pack_bf16x2(e[2], e[3]);
        u.z = pack_bf16x2(e[4], e[5]); u.w = pack_bf16x2(e[6], e[7]);
        *reinterpret_cast<uint4*>(prow + ((c ^ (t & 7)) << 4)) = u;
      }
      l_run += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ------------------------------ epilogue ------------------------------
    if (ok && n_tiles > 0) ok = mbar_wait(pv_done, uint32_t(n_tiles - 1) & 1, wctx, ST_TIMEOUT_MISC);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    // total row sum = sum of the two halves
    xch[512 + half * 128 + t] = l_run;
    __syncwarp();
    if (lane == 0) mbar_arrive(&xbar[qd]);
    ok = __all_sync(0xffffffffu, mbar_wait(&xbar[qd], xphase, wctx, ST_TIMEOUT_MISC)) && ok;
    const float l_tot = l_run + xch[512 + (half ^ 1) * 128 + t];
    const float inv_l = (l_tot > 0.f) ? 1.f / l_tot : 0.f;
    __nv_bfloat16* orow = p.O + (size_t(batch) * p.S + row) * p.ldo + head * D;
#pragma unroll 1
    for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
      uint32_t r[32];
      if (n_tiles > 0) {
        tmem_ld32(lane_addr + uint32_t(Cfg::O_COL + c * 32), r);
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
          *reinterpret_cast<uint4*>(orow + c * 32 + v4 * 8) = u;
        }
      }
    }
    if (half == 0 && ok && row < p.S && p.lse != nullptr) {
      const float m_eff = (m_run == -INFINITY) ? 0.f : m_run;
      p.lse[(size_t(batch) * p.Hq + head) * p.S + row] =
          (l_tot > 0.f) ? (m_eff * p.scale_log2 + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
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

// 4-D view {D-within-head, head, token-in-sequence, batch} of a packed [B*S, width] buffer
static int make_head_tmap3(CUtensorMap* out, const __nv_bfloat16* base, int B, int S, int heads, int D, int width,
                          int box_rows) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(heads), uint64_t(S), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(width) * 2, uint64_t(width) * 2 * uint64_t(S)};
  uint32_t box[4] = {64, 1, uint32_t(box_rows), 1};
  return make_tmap_nd_bf16(out, base, 4, dims, strides, box);
}

template <int D>
static int launch_fwd3(const __nv_bfloat16* qkv, int width, const AttnFwd3Params& p, cudaStream_t stream) {
  using Cfg = AttnFwd3Cfg<D>;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_head_tmap3(&tq, qkv, p.B, p.S, p.Hq, D, width, Cfg::BM))) return rc;
  if ((rc = make_head_tmap3(&tk, qkv + size_t(p.Hq) * D, p.B, p.S, p.Hkv, D, width, Cfg::BN))) return rc;
  if ((rc = make_head_tmap3(&tv, qkv + size_t(p.Hq + p.Hkv) * D, p.B, p.S, p.Hkv, D, width, Cfg::BN))) return rc;
  auto kern = flash_fwd3_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set = true;
  }
  dim3 grid((p.S + Cfg::BM - 1) / Cfg::BM, p.Hq, p.B);
  kern<<<grid, 320, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace zb

extern "C" int zb_flash_fwd3(const void* qkv, void* out, float* lse, int B, int S, int Hq, int Hkv, int D,
                            int causal, int window, float softmax_scale, int ldo, int* status,
                            cudaStream_t stream) {
  using namespace zb;
  if (B <= 0 || S <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) ZB_FAIL(-1, "attention: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  AttnFwd3Params p;
  p.O = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.window = window; p.causal = causal;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.ldo = ldo;
  p.status = status;
  const int width = (Hq + 2 * Hkv) * D;
  auto Q = static_cast<const __nv_bfloat16*>(qkv);
  if (D == 128) return launch_fwd3<128>(Q, width, p, stream);
  if (D == 64) return launch_fwd3<64>(Q, width, p, stream);
  ZB_FAIL(-1, "attention: head dim %d unsupported (64 or 128)", D);
}
