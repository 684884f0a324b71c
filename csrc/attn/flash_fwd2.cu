// Flash attention forward, two query tiles per CTA (256 query rows), sm_100a.
//
// Two independent softmax/MMA chains (A: rows [q0, q0+128), B: rows [q0+128, q0+256)) share
// the K/V tiles that one producer warp streams in by TMA.  Per chain and key tile j:
//     S = Q K_j^T           tcgen05.mma, SS form, fp32 in TMEM (128 columns)
//     P = exp2(S*c - m*c)   warps of the chain, one row per thread; P is written back as
//                           packed bf16 over the first 64 columns of S (tcgen05.st)
//     O += P V_j            tcgen05.mma, TS form: A = P straight from tensor memory
// so P never touches shared memory and the two chains keep the tensor pipe busy while the
// other one is in its softmax.  O is rescaled in TMEM only when a row maximum grew by more
// than 2^8 (the final normalisation absorbs the slack).
// Warps 0-3: softmax chain A, 4-7: softmax chain B, 8 / 9: MMA issuer of chain A / B (warp 8
// also owns the TMEM allocation), 10: TMA producer.  TMEM: S_A [0,128) S_B [128,256)
// O_A [256,256+D) O_B [384,384+D).  Same interface and layouts as flash_fwd.cu.
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

struct AttnFwd2Params {
  __nv_bfloat16* O;
  float* lse;
  int B, S, Hq, Hkv;
  int window, causal;
  float scale_log2;
  int ldo;
  int* status;
};

template <int D>
struct AttnFwd2Cfg {
  static constexpr int BM = 128, BN = 128;
  static constexpr int TILE_BYTES = 128 * D * 2;
  static constexpr int KV_STAGES = 2;
  static constexpr int SMEM_BYTES = 2 * TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 1024 + 256;
  static constexpr int THREADS = 352;
};

template <int D>
__global__ void __launch_bounds__(352, 1)
flash_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                  const __grid_constant__ CUtensorMap tmap_v, const AttnFwd2Params p) {
  using Cfg = AttnFwd2Cfg<D>;
  constexpr int BM = 128, BN = 128, STAGES = Cfg::KV_STAGES, DB = D / 64, BLK = 128 * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                // two tiles
  uint8_t* sK = sQ + 2 * Cfg::TILE_BYTES;            // STAGES tiles
  uint8_t* sV = sK + STAGES * Cfg::TILE_BYTES;       // STAGES tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + STAGES * Cfg::TILE_BYTES);
  uint64_t* q_full = bars;              // [2]
  uint64_t* k_full = bars + 2;          // [STAGES]
  uint64_t* k_empty = k_full + STAGES;  // [STAGES], 2 arrivals (one per chain)
  uint64_t* v_full = k_empty + STAGES;
  uint64_t* v_empty = v_full + STAGES;  // 2 arrivals
  uint64_t* s_full = v_empty + STAGES;  // [2]
  uint64_t* p_full = s_full + 2;        // [2], 4 arrivals
  uint64_t* o_done = p_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_pairs = (p.S + 2 * BM - 1) / (2 * BM);
  const int pair = n_pairs - 1 - int(blockIdx.x);  // heavy (late) tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int n_kv = (p.S + BN - 1) / BN;
  // key-tile range of each chain, and of the CTA (their union)
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
  const int j_lo = (hi[1] > lo[1]) ? min(lo[0], lo[1]) : lo[0];
  const int j_hi = max(hi[0], hi[1]);
  const int n_tiles = j_hi - j_lo;
  WaitCtx wctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int c = 0; c < 2; ++c) {
      mbar_init(&q_full[c], 1);
      mbar_init(&s_full[c], 1);
      mbar_init(&p_full[c], 4);
      mbar_init(&o_done[c], 1);
    }
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 2);
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

  if (warp == 10) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      for (int c = 0; c < 2; ++c) {
        if (hi[c] <= lo[c]) continue;
        mbar_expect_tx(&q_full[c], Cfg::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          tma_load_4d(sQ + c * Cfg::TILE_BYTES + b * BLK, &tmap_q, &q_full[c], b * 64, head, (2 * pair + c) * BM, batch);
      }
      for (int i = 0; i < n_tiles; ++i) {
        const int st = i % STAGES;
        const uint32_t ph = uint32_t(i / STAGES) & 1;
        const int kv0 = (j_lo + i) * BN;
        if (!mbar_wait(&k_empty[st], ph ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&k_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          tma_load_4d(sK + st * Cfg::TILE_BYTES + b * BLK, &tmap_k, &k_full[st], b * 64, kv_head, kv0, batch);
        if (!mbar_wait(&v_empty[st], ph ^ 1, wctx, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(&v_full[st], Cfg::TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DB; ++b)
          tma_load_4d(sV + st * Cfg::TILE_BYTES + b * BLK, &tmap_v, &v_full[st], b * 64, kv_head, kv0, batch);
      }
    }
  } else if (warp >= 8) {
    // ------------------------------ MMA issuer of chain c ------------------------------
    const int c = warp - 8;
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BM, BN, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(BM, D, false, true);
      const uint32_t s_col = tmem_base + uint32_t(c * 128);
      const uint32_t o_col = tmem_base + uint32_t(256 + c * 128);
      const bool active = hi[c] > lo[c];
      bool ok = true;
      if (active) ok = mbar_wait(&q_full[c], 0, wctx, ST_TIMEOUT_FULL);
      int used = 0;
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int st = i % STAGES;
        const uint32_t ph = uint32_t(i / STAGES) & 1;
        const int j = j_lo + i;
        if (!active || j < lo[c] || j >= hi[c]) {
          // this chain does not use the tile: just hand the stage back when it is loaded
          if (!mbar_wait(&k_full[st], ph, wctx, ST_TIMEOUT_FULL)) { ok = false; break; }
          mbar_arrive(&k_empty[st]);
          if (!mbar_wait(&v_full[st], ph, wctx, ST_TIMEOUT_FULL)) { ok = false; break; }
          mbar_arrive(&v_empty[st]);
          continue;
        }
        if (!mbar_wait(&k_full[st], ph, wctx, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + c * Cfg::TILE_BYTES), k_addr = smem_u32(sK + st * Cfg::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = uint32_t(kk / 4) * BLK + uint32_t(kk % 4) * 32;
          umma_f16_ss(s_col, umma_desc_kmajor(q_addr + off), umma_desc_kmajor(k_addr + off), idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[c]);
        if (!mbar_wait(&v_full[st], ph, wctx, ST_TIMEOUT_FULL)) { ok = false; break; }
        if (!mbar_wait(&p_full[c], uint32_t(used) & 1, wctx, ST_TIMEOUT_MISC)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + st * Cfg::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)
          umma_f16_ts(o_col, s_col + uint32_t(kk * 8), umma_desc_mnmajor(v_addr + kk * 16 * 128, BLK), idesc_o,
                      (used | kk) != 0 ? 1u : 0u);
        umma_commit(&v_empty[st]);
        ++used;
      }
      if (ok && active) umma_commit(&o_done[c]);
    }
  } else {
    // ------------------------------ softmax warps of chain c ------------------------------
    const int c = warp >> 2;
    const int t = threadIdx.x & 127;  // row inside the chain's query tile = TMEM lane
    const int q0 = (2 * pair + c) * BM;
    const int row = q0 + t;
    const uint32_t lane_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const uint32_t s_col = lane_addr + uint32_t(c * 128);
    const uint32_t o_col = lane_addr + uint32_t(256 + c * 128);
    const int my_tiles = max(hi[c] - lo[c], 0);
    float m_run = -INFINITY, l_run = 0.f;  // m_run in raw (unscaled) score units
    bool ok = true;
    for (int i = 0; i < my_tiles; ++i) {
      const int kv0 = (lo[c] + i) * BN;
      if (!__all_sync(0xffffffffu, mbar_wait(&s_full[c], uint32_t(i) & 1, wctx, ST_TIMEOUT_TMEM_FULL))) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (p.causal && kv0 + BN - 1 > q0) || (p.window > 0 && kv0 < q0 + BM - p.window) ||
                             (kv0 + BN > p.S);
      // pass 1: row maximum. All 128 columns are requested before the single wait, so the
      // TMEM round trip is paid once; four independent partial maxima keep the chains short.
      float tmax;
      {
        uint32_t r[4][32];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) tmem_ld32(s_col + uint32_t(ch * 32), r[ch]);
        tmem_wait_ld();
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (need_mask) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int col = kv0 + ch * 32 + k;
              const bool vis = (col < p.S) && (!p.causal || col <= row) && (p.window <= 0 || row - col < p.window);
              mx[ch] = fmaxf(mx[ch], vis ? __uint_as_float(r[ch][k]) : -INFINITY);
            }
        } else {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
#pragma unroll
            for (int k = 0; k < 32; ++k) mx[ch] = fmaxf(mx[ch], __uint_as_float(r[ch][k]));
        }
        tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      }
      // running maximum; O is rescaled only when it grew by more than 8 in log2 units
      if (i == 0) {
        m_run = tmax;
      } else {
        const bool need = (tmax - m_run) * p.scale_log2 > 8.f;
        if (__any_sync(0xffffffffu, need)) {
          float alpha = 1.f;
          if (need) {
            alpha = (m_run == -INFINITY) ? 0.f : exp2f((m_run - tmax) * p.scale_log2);
            m_run = tmax;
            l_run *= alpha;
          }
          // s_full(i) arrived => every MMA issued before it, including P V of tile i-1, is done
#pragma unroll
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
      const float m_eff = (m_run == -INFINITY) ? 0.f : m_run;
      const float neg_mc = -m_eff * p.scale_log2;
      // pass 2: P = exp2(S*c - m*c), packed bf16 pairs written over the first 64 columns of S.
      // Chunk c+1 is requested before chunk c is processed, so only the first TMEM round trip is
      // exposed; four independent partial sums keep the dependent-add chains short.
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      {
        uint32_t ra[32], rb[32];
        tmem_ld32(s_col, ra);
        tmem_wait_ld();
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t (&cur)[32] = (ch & 1) ? rb : ra;
          uint32_t (&nxt)[32] = (ch & 1) ? ra : rb;
          if (ch + 1 < 4) tmem_ld32(s_col + uint32_t((ch + 1) * 32), nxt);
          uint32_t pk[16];
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float e0 = exp2f(fmaf(__uint_as_float(cur[k]), p.scale_log2, neg_mc));
            float e1 = exp2f(fmaf(__uint_as_float(cur[k + 1]), p.scale_log2, neg_mc));
            if (need_mask) {
              const int c0 = kv0 + ch * 32 + k;
              e0 = ((c0 < p.S) && (!p.causal || c0 <= row) && (p.window <= 0 || row - c0 < p.window)) ? e0 : 0.f;
              e1 = ((c0 + 1 < p.S) && (!p.causal || c0 + 1 <= row) && (p.window <= 0 || row - c0 - 1 < p.window)) ? e1 : 0.f;
            }
            ls[(k >> 1) & 3] += e0 + e1;
            pk[k >> 1] = pack_bf16x2(e0, e1);
          }
          // chunk ch+1 (columns 32(ch+1)..) must have left TMEM before P overwrites columns
          // [16 ch, 16 ch + 16): for ch >= 1 those columns belong to chunks already consumed,
          // for ch == 0 they belong to chunk 0 itself
          if (ch + 1 < 4) tmem_wait_ld();
          tmem_st16(s_col + uint32_t(ch * 16), pk);
        }
      }
      const float lsum = (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tmem_wait_st();
      l_run += lsum;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[c]);
    }
    // ------------------------------ epilogue ------------------------------
    if (ok && my_tiles > 0) ok = mbar_wait(&o_done[c], 0, wctx, ST_TIMEOUT_MISC);
    ok = __all_sync(0xffffffffu, ok);
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
          (l_run > 0.f) ? (m_eff * p.scale_log2 + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
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

static int make_head_tmap2(CUtensorMap* out, const __nv_bfloat16* base, int B, int S, int heads, int D, int width) {
  uint64_t dims[4] = {uint64_t(D), uint64_t(heads), uint64_t(S), uint64_t(B)};
  uint64_t strides[3] = {uint64_t(D) * 2, uint64_t(width) * 2, uint64_t(width) * 2 * uint64_t(S)};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_nd_bf16(out, base, 4, dims, strides, box);
}

template <int D>
static int launch_fwd2(const __nv_bfloat16* qkv, int width, const AttnFwd2Params& p, cudaStream_t stream) {
  using Cfg = AttnFwd2Cfg<D>;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_head_tmap2(&tq, qkv, p.B, p.S, p.Hq, D, width))) return rc;
  if ((rc = make_head_tmap2(&tk, qkv + size_t(p.Hq) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  if ((rc = make_head_tmap2(&tv, qkv + size_t(p.Hq + p.Hkv) * D, p.B, p.S, p.Hkv, D, width))) return rc;
  auto kern = flash_fwd2_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set = true;
  }
  dim3 grid((p.S + 255) / 256, p.Hq, p.B);
  kern<<<grid, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace zb

extern "C" int zb_flash_fwd2(const void* qkv, void* out, float* lse, int B, int S, int Hq, int Hkv, int D,
                             int causal, int window, float softmax_scale, int ldo, int* status,
                             cudaStream_t stream) {
  using namespace zb;
  if (B <= 0 || S <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) ZB_FAIL(-1, "attention: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
  AttnFwd2Params p;
  p.O = static_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.window = window; p.causal = causal;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.ldo = ldo;
  p.status = status;
  const int width = (Hq + 2 * Hkv) * D;
  auto Q = static_cast<const __nv_bfloat16*>(qkv);
  if (D == 128) return launch_fwd2<128>(Q, width, p, stream);
  if (D == 64) return launch_fwd2<64>(Q, width, p, stream);
  ZB_FAIL(-1, "attention: head dim %d unsupported (64 or 128)", D);
}
