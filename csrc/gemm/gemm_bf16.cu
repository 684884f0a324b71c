// Persistent bf16 GEMM for sm_100a: C[M,N] = A * B^T (+ bias) (+ addend | += C).
//
//   * operands staged in shared memory by TMA (128-byte swizzle, never multicast),
//   * tcgen05.mma (kind::f16, M=128, N=BN, K=16) issued by one thread, fp32 accumulators
//     in tensor memory, two accumulator buffers so the epilogue of tile i overlaps the
//     main loop of tile i+1,
//   * warp roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2..5 =
//     epilogue (tcgen05.ld -> registers -> global).
//
// Operand layouts ("K-major" = the reduction dimension is contiguous):
//   A K-major : A stored [M, K] row-major (lda)        -- activations in fwd / dgrad
//   A MN-major: A stored [K, M] row-major (lda)        -- dY^T in wgrad
//   B K-major : B stored [N, K] row-major (ldb)        -- nn.Linear weight in fwd
//   B MN-major: B stored [K, N] row-major (ldb)        -- weight in dgrad, X in wgrad
//
// Plays the role of the cuBLAS calls behind nn.Linear and its autograd in the reference
// (models/llama_simple.py:206-221, models/llama_v2.py:222-229).
#include "../common/host.h"
#include "../common/ptx.cuh"
#include "gemm_common.cuh"

namespace zb {

template <int BN>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int BK = 64;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int NUM_THREADS = 192;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, bool A_MN, bool B_MN, bool FUSED_AG>
__global__ void __launch_bounds__(FUSED_AG ? 320 : 192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p, const AgParams ag) {
  using Cfg = GemmCfg<BN>;
  constexpr int BM = Cfg::BM, BK = Cfg::BK, STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tmem_full = bars + 2 * STAGES;
  uint64_t* tmem_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM;
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
      mbar_init(&tmem_empty[i], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM;
        const int n0 = (tile / tiles_m) * BN;
        if (!zb_in_bounds(m0 < p.M && n0 < p.N && tile >= 0, p.status, 1)) break;
        if (p.gate_flags != nullptr) {
          const long b0 = p.gate_base + long(n0) * p.gate_row_bytes;
          const long b1 = p.gate_base + long(min(n0 + BN, p.N)) * p.gate_row_bytes - 1;
          const long i0 = (b0 / p.gate_shard_bytes) * p.gate_cps + (b0 % p.gate_shard_bytes) / p.gate_chunk_bytes;
          const long i1 = (b1 / p.gate_shard_bytes) * p.gate_cps + (b1 % p.gate_shard_bytes) / p.gate_chunk_bytes;
          for (long c = i0; c <= i1 && ok; ++c) {
            if (int(c / p.gate_cps) == p.gate_self) continue;
            ok = flag_wait_ge(p.gate_flags + c, p.gate_epoch, ZB_WAIT_NS, p.status, ST_TIMEOUT_FLAG);
          }
          if (!ok) {
            *abort_flag = 1;
            break;
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, wctx, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full[stage], Cfg::STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (BK * 128), &tmap_a, &full[stage], m0 + j * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (BK * 128), &tmap_b, &full[stage], n0 + j * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t use = uint32_t(local >> 1);
        if (!mbar_wait(&tmem_empty[buf], (use & 1) ^ 1, wctx, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full[stage], phase, wctx, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            uint64_t da = A_MN ? umma_desc_mnmajor(sa + kk * 16 * 128, BK * 128)
                               : umma_desc_kmajor(sa + kk * 32);
            uint64_t db = B_MN ? umma_desc_mnmajor(sb + kk * 16 * 128, BK * 128)
                               : umma_desc_kmajor(sb + kk * 32);
            umma_f16_ss(d_tmem, da, db, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(&tmem_full[buf]);
      }
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const EpilogueCfg ecfg = epilogue_cfg(p);
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int m0 = (tile % tiles_m) * BM;
      const int n0 = (tile / tiles_m) * BN;
      const int buf = local & 1;
      const uint32_t use = uint32_t(local >> 1);
      if (!__all_sync(0xffffffffu, mbar_wait(&tmem_full[buf], use & 1, wctx, ST_TIMEOUT_TMEM_FULL))) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(buf * BN + c * 32), r);
        tmem_wait_ld();
        if (!row_ok) continue;
        epilogue_store_chunk(p, ecfg, row, col0, r);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
  }

  if (FUSED_AG && warp >= 6) {
    // ------------------------------ all-gather copy warps ------------------------------
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
      for (; i + 7 * 128 < end; i += 8 * 128) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = ld_v4_relaxed_sys(src + i + u * 128);
#pragma unroll
        for (int u = 0; u < 8; ++u) dst[i + u * 128] = v[u];
      }
      for (; i < end; i += 128) dst[i] = ld_v4_relaxed_sys(src + i);
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (ct == 0) st_release_sys(ag.chunk_flags + peer * ag.cps + c, ag.epoch);
    }
    if (!ok) *abort_flag = 1;
  }

  // ------------------------------ teardown ------------------------------
  __syncwarp();
  if (*abort_flag) {
    // copies may still be in flight towards this CTA's shared memory: give them time
    // to land before the CTA exits (bounded).
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, bool FUSED_AG>
static int launch_gemm(const void* A, const void* B, const GemmParams& p, const AgParams& ag, int lda, int ldb,
                       int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap ta, tb;
  int rc;
  if (!A_MN) rc = make_tmap_2d_bf16(&ta, A, p.M, p.K, lda, Cfg::BM, 64);
  else rc = make_tmap_2d_bf16(&ta, A, p.K, p.M, lda, 64, 64);
  if (rc) return rc;
  if (!B_MN) rc = make_tmap_2d_bf16(&tb, B, p.N, p.K, ldb, BN, 64);
  else rc = make_tmap_2d_bf16(&tb, B, p.K, p.N, ldb, 64, 64);
  if (rc) return rc;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, FUSED_AG>;
  static bool attr_set = false;
  if (!attr_set) {
    ZB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set = true;
  }
  const int tiles = ((p.M + Cfg::BM - 1) / Cfg::BM) * ((p.N + BN - 1) / BN);
  int ctas = num_sms();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (tiles < ctas) ctas = tiles;
  kern<<<ctas, FUSED_AG ? 320 : Cfg::NUM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, p, ag);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // namespace zb

extern "C" {

static void fill_gemm_params(zb::GemmParams& p, void* C, int M, int N, int K, int ldc, const void* bias,
                             const void* addend, int ld_addend, int flags, int* status) {
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
}

static int pick_bn(int M, int N, int bn) {
  if (bn == 128 || bn == 256) return bn;
  long tiles256 = long((M + 127) / 128) * ((N + 255) / 256);
  bn = (tiles256 >= zb::num_sms() || (N > 256 && tiles256 * 2 > zb::num_sms() * 3)) ? 256 : 128;
  if (N <= 128) bn = 128;
  return bn;
}

// Returns 0 on success; on failure zb_last_error() describes it. `status` is a device
// int the kernel writes a non-zero code to if one of its bounded waits ran out.
int zb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                 int ldc, int a_mn_major, int b_mn_major, const void* bias, const void* addend,
                 int ld_addend, int flags, int bn, int max_ctas, int* status, cudaStream_t stream) {
  using namespace zb;
  if (M <= 0 || N <= 0 || K <= 0) ZB_FAIL(-1, "gemm: empty problem %d x %d x %d", M, N, K);
  GemmParams p;
  fill_gemm_params(p, C, M, N, K, ldc, bias, addend, ld_addend, flags, status);
  AgParams ag = {};
  bn = pick_bn(M, N, bn);
#define ZB_DISPATCH(BN_)                                                                          \
  if (!a_mn_major && !b_mn_major) return launch_gemm<BN_, false, false, false>(A, B, p, ag, lda, ldb, max_ctas, stream); \
  if (!a_mn_major && b_mn_major) return launch_gemm<BN_, false, true, false>(A, B, p, ag, lda, ldb, max_ctas, stream);   \
  if (a_mn_major && b_mn_major) return launch_gemm<BN_, true, true, false>(A, B, p, ag, lda, ldb, max_ctas, stream);     \
  return launch_gemm<BN_, true, false, false>(A, B, p, ag, lda, ldb, max_ctas, stream);
  if (bn == 256) { ZB_DISPATCH(256) }
  ZB_DISPATCH(128)
#undef ZB_DISPATCH
}

// All-gather fused with the GEMM that first consumes the gathered weights:
//   C[M,N] = A[M,K] * B[N,K]^T (+bias)(+addend), B = a [N,K] weight inside the unit's flat
//   unsharded buffer `full` (byte offset b_offset), whose remote shards this same kernel pulls
//   from the peers (shard_ptrs, peer-mapped) while the tiles of already-present rows run.
// chunk_flags: local int[R*cps], cps = ceil(shard_bytes / chunk_bytes); a chunk is complete
// when its flag equals `epoch`. version_flags: local int[R] the peers write their shard epoch to.
int zb_ag_gemm_bf16(const void* A, void* full, long b_offset_bytes, void* C, int M, int N, int K, int lda, int ldc,
                    const void* bias, const void* addend, int ld_addend, int flags, const void* const* shard_ptrs,
                    int R, int r, long shard_bytes, int chunk_bytes, int* chunk_flags, int epoch,
                    const int* version_flags, int need_version, int* status, cudaStream_t stream) {
  using namespace zb;
  if (M <= 0 || N <= 0 || K <= 0) ZB_FAIL(-1, "ag_gemm: empty problem %d x %d x %d", M, N, K);
  if (R < 2 || R > AG_MAX_R) ZB_FAIL(-1, "ag_gemm: group size %d unsupported (2..%d)", R, AG_MAX_R);
  if (shard_bytes % 16 || chunk_bytes % 2048 || chunk_bytes <= 0) ZB_FAIL(-1, "ag_gemm: bad shard/chunk size");
  GemmParams p;
  fill_gemm_params(p, C, M, N, K, ldc, bias, addend, ld_addend, flags, status);
  AgParams ag;
  for (int i = 0; i < R; ++i) ag.src[i] = static_cast<const uint4*>(shard_ptrs[i]);
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
  const int bn = pick_bn(M, N, 0);
  if (bn == 256) return launch_gemm<256, false, false, true>(A, B, p, ag, lda, K, 0, stream);
  return launch_gemm<128, false, false, true>(A, B, p, ag, lda, K, 0, stream);
}

const char* zb_last_error() { return zb::last_error_buf(); }

}  // extern "C"
