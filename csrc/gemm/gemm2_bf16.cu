// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 with a 256 x 256 output tile per pair.
//
// Two CTAs of a cluster (2,1,1) share one tile: each holds 128 rows of A and of the fp32
// accumulators (its own tensor memory) and loads HALF of the B tile (128 of the 256 rows);
// the MMA issued by the leader CTA reads A and B from both CTAs' shared memory.  Per k-block a
// pair moves 64 KB for 256x256x64 MACs, 1.5x the arithmetic intensity of the single-CTA
// 128x256 kernel, which is what the L2 -> SM path needs at tensor-core rate.
//   * every TMA load is issued by the CTA that receives the data, WITHOUT cluster multicast;
//     its mbarrier completion is routed to the leader's barrier (cta_group::2 form),
//   * tcgen05.commit with cluster multicast hands stages / accumulators back to both CTAs,
//   * warp roles per CTA: 0 = TMA producer, 1 = MMA issuer (leader only) + TMEM owner,
//     2..5 = epilogue for the CTA's own 128 rows.
// Operand layouts and epilogue options are those of gemm_bf16.cu.
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "gemm_common.cuh"
#include <type_traits>

namespace zb {

constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}
// arrive on the barrier at the same shared-memory offset in CTA `cta` of the cluster
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t cta) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}" ::"r"(smem_u32(bar)),
      "r"(cta)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint64_t* leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(leader_bar) & PEER_BIT_MASK), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const void* tmap, uint64_t* leader_bar, int x, int y,
                                                 int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(leader_bar) & PEER_BIT_MASK), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0), "r"(0),
        "r"(0), "r"(0), "r"(0)
      : "memory");
}
// arrives (once all MMAs issued so far are complete) on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(uint16_t(3))
      : "memory");
}

struct Gemm2Cfg {
  static constexpr int BM = 256;   // per pair; 128 per CTA
  static constexpr int BN = 256;   // per pair; each CTA loads 128 rows of B
  static constexpr int BK = 64;
  static constexpr int A_BYTES = 128 * BK * 2;
  static constexpr int B_BYTES = 128 * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

struct Gemm2Extra {
  int a_3d, b_3d;  // MN-major operand fetched with one 3-D TMA box {64, BK, 2} instead of two 2-D boxes
};

// SCATTER: the epilogue sends every output row to the staging slot of the rank that owns it in a
// row-wise reduce-scatter (plain stores over NVLink, tile by tile while the main loop goes on) and
// the last CTA raises the arrival flags; the owners add the slots up (csrc/comm/tp_rs.cu).
// FUSED_AG (Params = GemmAgParams): four more warps per CTA pull the peers' parameter shards into the local
// unsharded buffer while the tiles whose B rows are already present run; each CTA's producer waits for the
// chunks that cover its own 128 rows of B.
template <bool A_MN, bool B_MN, typename Params = GemmParams>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(std::is_same<Params, GemmAgParams>::value ? 320 : 192, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const Params p, const Gemm2Extra ex) {
  using Cfg = Gemm2Cfg;
  constexpr bool SCATTER = std::is_same<Params, GemmScatterParams>::value;
  constexpr bool ACCPF = std::is_same<Params, GemmAccPrefetchParams>::value;
  constexpr bool FUSED_AG = std::is_same<Params, GemmAgParams>::value;
  constexpr int BK = Cfg::BK, STAGES = Cfg::STAGES, BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;                          // leader's copy is the one in use
  uint64_t* empty = bars + STAGES;                // each CTA waits on its own
  uint64_t* tmem_full = bars + 2 * STAGES;        // [2], each CTA waits on its own
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;   // [2], leader's copy, 8 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (p.M + Cfg::BM - 1) / Cfg::BM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  WaitCtx wctx{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % tiles_m) * Cfg::BM + int(cta) * 128;
        const int n0 = (tile / tiles_m) * BN + int(cta) * 128;
        // (the second CTA's half may start past the edge of a ragged tile: its loads then read the fill value)
        if (!zb_in_bounds(m0 - int(cta) * 128 < p.M && n0 - int(cta) * 128 < p.N && tile >= 0, p.status, 1)) break;
        if constexpr (FUSED_AG) {
          if (p.gate_flags != nullptr && n0 < p.N) {
            // rows [n0, n0 + 128) of B inside the flat buffer: wait for every chunk of a peer's shard they touch
            const long b0 = p.gate_base + long(n0) * p.gate_row_bytes;
            const long b1 = p.gate_base + long(min(n0 + 128, p.N)) * p.gate_row_bytes - 1;
            const long i0 = (b0 / p.gate_shard_bytes) * p.gate_cps + (b0 % p.gate_shard_bytes) / p.gate_chunk_bytes;
            const long i1 = (b1 / p.gate_shard_bytes) * p.gate_cps + (b1 % p.gate_shard_bytes) / p.gate_chunk_bytes;
            for (long c = i0; c <= i1 && ok; ++c) {
              if (int(c / p.gate_cps) == p.gate_self) continue;
              ok = flag_wait_ge(p.gate_flags + c, p.gate_epoch, ZB_WAIT_NS, p.status, ST_TIMEOUT_FLAG);
            }
            if (!ok) { *abort_flag = 1; break; }
            asm volatile("fence.proxy.async.global;" ::: "memory");   // the gathered rows were written with plain stores
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, wctx, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          if (leader) mbar_expect_tx(&full[stage], 2 * Cfg::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmap_a, &full[stage], kb * BK, m0);
          } else if (ex.a_3d) {
            tma_load_3d_pair(sa, &tmap_a, &full[stage], 0, kb * BK, m0 >> 6);
          } else {
            tma_load_2d_pair(sa, &tmap_a, &full[stage], m0, kb * BK);
            tma_load_2d_pair(sa + BK * 128, &tmap_a, &full[stage], m0 + 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, &full[stage], kb * BK, n0);
          } else if (ex.b_3d) {
            tma_load_3d_pair(sb, &tmap_b, &full[stage], 0, kb * BK, n0 >> 6);
          } else {
            tma_load_2d_pair(sb, &tmap_b, &full[stage], n0, kb * BK);
            tma_load_2d_pair(sb + BK * 128, &tmap_b, &full[stage], n0 + 64, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(256, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int buf = local & 1;
        const uint32_t use = uint32_t(local >> 1);
        if (!mbar_wait(&tmem_empty[buf], (use & 1) ^ 1, wctx, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, wctx, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            uint64_t da = A_MN ? umma_desc_mnmajor(sa + kk * 16 * 128, BK * 128) : umma_desc_kmajor(sa + kk * 32);
            uint64_t db = B_MN ? umma_desc_mnmajor(sb + kk * 16 * 128, BK * 128) : umma_desc_kmajor(sb + kk * 32);
            umma_f16_ss_pair(d_tmem, da, db, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[buf]);
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue (own 128 rows) ------------------------------
    const int q = warp & 3;
    const EpilogueCfg ecfg = epilogue_cfg(p);
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const int m0 = (tile % tiles_m) * Cfg::BM + int(cta) * 128;
      const int n0 = (tile / tiles_m) * BN;
      const int buf = local & 1;
      const uint32_t use = uint32_t(local >> 1);
      if constexpr (ACCPF) {
        // bf16 C += result without bias / addend / activation (checked on the host): request this thread's whole
        // old C row of the tile now; the loads complete while the tile's main loop is still running
        const int row = m0 + q * 32 + lane;
        const bool row_ok = row < p.M;
        const bool fast = row_ok && ecfg.vec_ok && n0 + BN <= p.N;
        uint4 oldc[BN / 8];
        __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(p.C) + size_t(row_ok ? row : 0) * p.ldc + n0;
        if (fast) {
#pragma unroll
          for (int j = 0; j < BN / 8; ++j) oldc[j] = reinterpret_cast<const uint4*>(crow)[j];
        }
        if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[buf], use & 1, wctx, ST_TIMEOUT_TMEM_FULL))) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 < p.N) {
            uint32_t r[32];
            tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * BN + c * 32), r);
            tmem_wait_ld();
            if (fast) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint4 a = oldc[c * 4 + j];
                const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
                uint4 o;
                o.x = pack_bf16x2(__uint_as_float(r[j * 8 + 0]) + f0.x, __uint_as_float(r[j * 8 + 1]) + f0.y);
                o.y = pack_bf16x2(__uint_as_float(r[j * 8 + 2]) + f1.x, __uint_as_float(r[j * 8 + 3]) + f1.y);
                o.z = pack_bf16x2(__uint_as_float(r[j * 8 + 4]) + f2.x, __uint_as_float(r[j * 8 + 5]) + f2.y);
                o.w = pack_bf16x2(__uint_as_float(r[j * 8 + 6]) + f3.x, __uint_as_float(r[j * 8 + 7]) + f3.y);
                reinterpret_cast<uint4*>(crow)[c * 4 + j] = o;
              }
            } else if (row_ok) {
              epilogue_store_chunk(p, ecfg, row, col0, r);
            }
          }
        }
      } else {
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[buf], use & 1, wctx, ST_TIMEOUT_TMEM_FULL))) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      __nv_bfloat16* crow = nullptr;   // SCATTER: this thread's destination row
      if constexpr (SCATTER) if (row_ok) {
        const int owner = row / p.sc_rows;
        crow = static_cast<__nv_bfloat16*>(p.sc_dst[owner]) + size_t(row - owner * p.sc_rows) * p.ldc;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * BN + c * 32), r);
        tmem_wait_ld();
        if (!row_ok) continue;
        if constexpr (SCATTER) epilogue_scatter_chunk(crow, col0, p.N, ecfg.vec_ok, r);
        else epilogue_store_chunk(p, ecfg, row, col0, r);
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(&tmem_empty[buf], 0);
    }
    if constexpr (SCATTER) __threadfence_system();   // this thread's rows are visible to their owners before the flags
  }

  if constexpr (FUSED_AG) if (warp >= 6) {
    // ------------------------------ all-gather copy warps ------------------------------
    const AgParams& ag = p.ag;
    const int ct = threadIdx.x - 192;  // 0..127
    __shared__ int s_peer_ok;
    const int total = (ag.R - 1) * ag.cps;
    const long chunk16 = ag.chunk_bytes / 16;
    const long shard16 = ag.shard_bytes / 16;
    int checked_peer = -1;
    bool ok = true;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      // ascending chunk order inside each peer, peers visited starting after this rank
      const int c = w / (ag.R - 1);
      const int pi = w % (ag.R - 1);
      const int peer = (ag.r + 1 + pi) % ag.R;
      if (peer != checked_peer) {
        if (ct == 0)
          s_peer_ok = flag_wait_ge(ag.version_flags + peer, ag.need_version, ZB_WAIT_NS, p.status, ST_TIMEOUT_FLAG) ? 1 : 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        ok = s_peer_ok != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        checked_peer = peer;
        if (!ok) break;
      }
      const long beg = long(c) * chunk16;
      const long end = min(beg + chunk16, shard16);
      if (!zb_in_bounds(peer >= 0 && peer < ag.R && peer != ag.r && beg >= 0 && end <= shard16 && beg <= end, p.status, 3)) break;
      if (!zb_in_bounds(peer * ag.cps + c < ag.R * ag.cps && c >= 0, p.status, 4)) break;
      const uint4* src = ag.src[peer];
      uint4* dst = ag.dst + long(peer) * shard16;
      long i = beg + ct;
      // Software-pipelined copy: the 8 requests of the next batch are issued before the 8 values of the current one are
      // stored, so a thread always has 8 - 16 peer loads of 16 bytes in flight (up to 32 KiB per CTA, 4.7 MB per GPU)
      // instead of draining to zero between batches.
      constexpr int UB = 8;
      const long step = long(UB) * 128;
      if (i + (UB - 1) * 128 < end) {
        uint4 cur[UB], nxt[UB];
#pragma unroll
        for (int u = 0; u < UB; ++u) cur[u] = ld_v4_relaxed_sys(src + i + u * 128);
        for (; i + step + (UB - 1) * 128 < end; i += step) {
#pragma unroll
          for (int u = 0; u < UB; ++u) nxt[u] = ld_v4_relaxed_sys(src + i + step + u * 128);
#pragma unroll
          for (int u = 0; u < UB; ++u) dst[i + u * 128] = cur[u];
#pragma unroll
          for (int u = 0; u < UB; ++u) cur[u] = nxt[u];
        }
#pragma unroll
        for (int u = 0; u < UB; ++u) dst[i + u * 128] = cur[u];
        i += step;
      }
      for (; i < end; i += 128) dst[i] = ld_v4_relaxed_sys(src + i);
      // the rows go from these stores (generic proxy) to the TMA loads of some CTA's producer (async proxy)
      __threadfence();
      asm volatile("fence.proxy.async.global;" ::: "memory");
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ct == 0) st_release_sys(ag.chunk_flags + peer * ag.cps + c, ag.epoch);
    }
    if (!ok) *abort_flag = 1;
  }

  // ------------------------------ teardown ------------------------------
  __syncwarp();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();  // the leader's MMAs read the peer's shared memory: leave together
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
  if constexpr (SCATTER) if (threadIdx.x == 0) {
    // last CTA of the grid: every row has been stored and fenced; tell the owners (not after a timeout:
    // the status word is then non-zero and the owners' bounded wait reports it)
    if (atomicAdd(p.sc_counter, 1u) == gridDim.x - 1) {
      __threadfence_system();
      if (*reinterpret_cast<volatile int*>(p.status) == 0)
        for (int q = 0; q < p.sc_R; ++q) st_release_sys(p.sc_flags[q] + p.sc_flag_index, p.sc_epoch);
      *p.sc_counter = 0u;
    }
  }
}

// 3-D view of an MN-major operand stored [K rows, MN cols]: {64 within a block, K, MN/64 blocks}
static int make_tmap_mn3d(CUtensorMap* out, const void* base, uint64_t krows, uint64_t mn, uint64_t ld) {
  uint64_t dims[3] = {64, krows, mn / 64};
  uint64_t strides[2] = {ld * 2, 128};
  uint32_t box[3] = {64, 64, 2};
  return make_tmap_nd_bf16(out, base, 3, dims, strides, box);
}

template <bool A_MN, bool B_MN, typename Params = GemmParams>
static int launch_gemm2(const void* A, const void* B, const Params& p, int lda, int ldb, int max_ctas,
                        cudaStream_t stream) {
  using Cfg = Gemm2Cfg;
  CUtensorMap ta, tb;
  Gemm2Extra ex = {0, 0};
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(&ta, A, p.M, p.K, lda, 128, 64);
  else if (p.M % 64 == 0) { rc = make_tmap_mn3d(&ta, A, p.K, p.M, lda); ex.a_3d = 1; }
  else rc = make_tmap_2d_bf16(&ta, A, p.K, p.M, lda, 64, 64);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tb, B, p.N, p.K, ldb, 128, 64);
  else if (p.N % 64 == 0) { rc = make_tmap_mn3d(&tb, B, p.K, p.N, ldb); ex.b_3d = 1; }
  else rc = make_tmap_2d_bf16(&tb, B, p.K, p.N, ldb, 64, 64);
  if (rc) return rc;
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, Params>;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set = true;
  }
  const int tiles = ((p.M + Cfg::BM - 1) / Cfg::BM) * ((p.N + Cfg::BN - 1) / Cfg::BN);
  int pairs = num_sms() / 2;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (tiles < pairs) pairs = tiles;
  kern<<<2 * pairs, std::is_same<Params, GemmAgParams>::value ? 320 : 192, Cfg::SMEM_BYTES, stream>>>(ta, tb, p, ex);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace zb

extern "C" int zb_gemm2_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                             int a_mn_major, int b_mn_major, const void* bias, const void* addend, int ld_addend,
                             int flags, int max_ctas, int* status, cudaStream_t stream) {
  using namespace zb;
  if (M <= 0 || N <= 0 || K <= 0) ZB_FAIL(-1, "gemm2: empty problem %d x %d x %d", M, N, K);
  GemmParams p;
  p.C = C;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.addend = static_cast<const __nv_bfloat16*>(addend);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ld_addend = ld_addend;
  p.flags = flags;
  p.status = status;
  p.gate_flags = nullptr;
  p.gate_epoch = 0;
  p.gate_base = 0; p.gate_row_bytes = 0; p.gate_shard_bytes = 1;
  p.gate_chunk_bytes = 1; p.gate_cps = 1; p.gate_self = -1;
  if (!a_mn_major && !b_mn_major) return launch_gemm2<false, false>(A, B, p, lda, ldb, max_ctas, stream);
  if (!a_mn_major && b_mn_major) return launch_gemm2<false, true>(A, B, p, lda, ldb, max_ctas, stream);
  if (a_mn_major && b_mn_major) return launch_gemm2<true, true>(A, B, p, lda, ldb, max_ctas, stream);
  return launch_gemm2<true, false>(A, B, p, lda, ldb, max_ctas, stream);
}

// C = A @ B^T (b_mn_major: A @ B) with the output rows scattered for a row-wise reduce-scatter over
// R ranks: rows [q * M / R, (q + 1) * M / R) go to dst_ptrs[q] (this rank's bf16 staging slot in rank
// q's memory, [M / R, N] with row stride ldc); when the grid is done `epoch` is stored to
// flag_ptrs[q][flag_index] for every q.  A: [M, K] K-major.  counter: zeroed device int.
extern "C" int zb_gemm2_rs_bf16(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int ldc,
                                int b_mn_major, void* const* dst_ptrs, int* const* flag_ptrs, int R, int flag_index,
                                int epoch, unsigned int* counter, int max_ctas, int* status, cudaStream_t stream) {
  using namespace zb;
  if (M <= 0 || N <= 0 || K <= 0) ZB_FAIL(-1, "gemm2_rs: empty problem %d x %d x %d", M, N, K);
  if (R < 1 || R > 8 || M % R != 0) ZB_FAIL(-1, "gemm2_rs: %d rows do not split over %d ranks (1..8)", M, R);
  GemmScatterParams p;
  p.C = nullptr;
  p.bias = nullptr; p.addend = nullptr;
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ld_addend = 0;
  p.flags = 0;
  p.status = status;
  p.gate_flags = nullptr;
  p.gate_epoch = 0;
  p.gate_base = 0; p.gate_row_bytes = 0; p.gate_shard_bytes = 1;
  p.gate_chunk_bytes = 1; p.gate_cps = 1; p.gate_self = -1;
  for (int q = 0; q < 8; ++q) { p.sc_dst[q] = nullptr; p.sc_flags[q] = nullptr; }
  for (int q = 0; q < R; ++q) {
    if (reinterpret_cast<uintptr_t>(dst_ptrs[q]) & 15) ZB_FAIL(-1, "gemm2_rs: destination %d not 16-byte aligned", q);
    p.sc_dst[q] = dst_ptrs[q];
    p.sc_flags[q] = flag_ptrs[q];
  }
  p.C = dst_ptrs[0];   // alignment of the vector path is judged on a destination
  p.sc_rows = M / R; p.sc_R = R; p.sc_flag_index = flag_index; p.sc_epoch = epoch; p.sc_counter = counter;
  if (b_mn_major) return launch_gemm2<false, true, GemmScatterParams>(A, B, p, lda, ldb, max_ctas, stream);
  return launch_gemm2<false, false, GemmScatterParams>(A, B, p, lda, ldb, max_ctas, stream);
}

// C (bf16) += A @ B^T with the old C tile requested before the tile's accumulators are ready (candidate for the
// weight-gradient GEMMs).  Same operand conventions as zb_gemm2_bf16; only bf16 accumulation without bias,
// addend or activation takes the prefetching kernel, anything else is forwarded to zb_gemm2_bf16.
extern "C" int zb_gemm2_accpf_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                   int ldc, int a_mn_major, int b_mn_major, const void* bias, const void* addend,
                                   int ld_addend, int flags, int max_ctas, int* status, cudaStream_t stream) {
  using namespace zb;
  if (flags != GEMM_ACCUMULATE || bias != nullptr || addend != nullptr)
    return zb_gemm2_bf16(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, bias, addend, ld_addend, flags,
                         max_ctas, status, stream);
  if (M <= 0 || N <= 0 || K <= 0) ZB_FAIL(-1, "gemm2: empty problem %d x %d x %d", M, N, K);
  GemmAccPrefetchParams p;
  p.C = C;
  p.bias = nullptr; p.addend = nullptr;
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ld_addend = 0;
  p.flags = flags;
  p.status = status;
  p.gate_flags = nullptr;
  p.gate_epoch = 0;
  p.gate_base = 0; p.gate_row_bytes = 0; p.gate_shard_bytes = 1;
  p.gate_chunk_bytes = 1; p.gate_cps = 1; p.gate_self = -1;
  if (!a_mn_major && !b_mn_major) return launch_gemm2<false, false, GemmAccPrefetchParams>(A, B, p, lda, ldb, max_ctas, stream);
  if (!a_mn_major && b_mn_major) return launch_gemm2<false, true, GemmAccPrefetchParams>(A, B, p, lda, ldb, max_ctas, stream);
  if (a_mn_major && b_mn_major) return launch_gemm2<true, true, GemmAccPrefetchParams>(A, B, p, lda, ldb, max_ctas, stream);
  return launch_gemm2<true, false, GemmAccPrefetchParams>(A, B, p, lda, ldb, max_ctas, stream);
}


// All-gather fused with the GEMM that first consumes the gathered weights, on the 2-CTA core
// (same contract as zb_ag_gemm_bf16 in gemm_bf16.cu): C[M,N] = A[M,K] * B[N,K]^T (+bias)(+addend),
// B = a [N,K] weight inside the unit's flat unsharded buffer `full` at byte offset b_offset_bytes.
extern "C" int zb_ag_gemm2_bf16(const void* A, void* full, long b_offset_bytes, void* C, int M, int N, int K, int lda,
                                int ldc, const void* bias, const void* addend, int ld_addend, int flags,
                                const void* const* shard_ptrs, int R, int r, long shard_bytes, int chunk_bytes,
                                int* chunk_flags, int epoch, const int* version_flags, int need_version, int* status,
                                cudaStream_t stream) {
  using namespace zb;
  if (M <= 0 || N <= 0 || K <= 0) ZB_FAIL(-1, "ag_gemm2: empty problem %d x %d x %d", M, N, K);
  if (R < 2 || R > AG_MAX_R) ZB_FAIL(-1, "ag_gemm2: group size %d unsupported (2..%d)", R, AG_MAX_R);
  if (shard_bytes % 16 || chunk_bytes % 2048 || chunk_bytes <= 0) ZB_FAIL(-1, "ag_gemm2: bad shard/chunk size");
  if (b_offset_bytes % 16 || (long(K) * 2) % 16) ZB_FAIL(-1, "ag_gemm2: weight offset / row size not 16-byte aligned");
  GemmAgParams p;
  p.C = C;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.addend = static_cast<const __nv_bfloat16*>(addend);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ld_addend = ld_addend;
  p.flags = flags;
  p.status = status;
  AgParams& ag = p.ag;
  for (int i = 0; i < AG_MAX_R; ++i) ag.src[i] = i < R ? static_cast<const uint4*>(shard_ptrs[i]) : nullptr;
  ag.dst = static_cast<uint4*>(full);
  ag.shard_bytes = shard_bytes;
  ag.R = R; ag.r = r;
  ag.chunk_bytes = chunk_bytes;
  ag.cps = int((shard_bytes + chunk_bytes - 1) / chunk_bytes);
  ag.chunk_flags = chunk_flags;
  ag.epoch = epoch;
  ag.version_flags = version_flags;
  ag.need_version = need_version;
  p.gate_flags = chunk_flags;
  p.gate_epoch = epoch;
  p.gate_base = b_offset_bytes;
  p.gate_row_bytes = long(K) * 2;
  p.gate_shard_bytes = shard_bytes;
  p.gate_chunk_bytes = chunk_bytes;
  p.gate_cps = ag.cps;
  p.gate_self = r;
  const void* B = static_cast<const char*>(full) + b_offset_bytes;
  return launch_gemm2<false, false, GemmAgParams>(A, B, p, lda, K, 0, stream);
}
