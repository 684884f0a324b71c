// Shared pieces of the GEMM kernels: launch parameters and the epilogue that turns one
// 32-column chunk of fp32 accumulators (one output row per thread) into stored output:
// (+ bias) (activation) (+ addend) (+= C), bf16 or fp32, 16-byte stores when aligned.
#pragma once
#include "../common/ptx.cuh"

namespace zb {

enum : int {
  GEMM_OUT_F32 = 1,     // C is fp32 (else bf16)
  GEMM_ACCUMULATE = 2,  // C += result (read-modify-write in C's dtype, fp32 add)
  GEMM_GELU = 4,        // tanh-GELU applied after bias (forward of GPT-style MLPs)
  GEMM_RELU = 8,
};

struct GemmParams {
  void* C;
  const __nv_bfloat16* bias;    // [N] or nullptr
  const __nv_bfloat16* addend;  // [M, ld_addend] bf16 or nullptr (e.g. residual)
  int M, N, K;
  int ldc, ld_addend;
  int flags;
  int* status;
  // optional arrival gating of B tiles (all-gather fused GEMM): B lives inside a flat
  // unsharded parameter buffer that is being filled shard by shard, chunk by chunk. Before
  // loading rows [n0, n_end] of B the producer waits until the flag of every chunk that
  // overlaps bytes [gate_base + n0*row_bytes, gate_base + (n_end+1)*row_bytes) of the flat
  // buffer is >= gate_epoch. Flag index of flat byte b: (b / shard_bytes) * cps +
  // (b % shard_bytes) / chunk_bytes; the rank's own shard needs no wait. nullptr = off.
  const int* gate_flags;
  int gate_epoch;
  long gate_base, gate_row_bytes, gate_shard_bytes;
  int gate_chunk_bytes, gate_cps, gate_self;
};


// Row scatter of the output (GEMM fused with the send half of a reduce-scatter over rows; used by
// the kernels instantiated with this parameter type): output row m goes to row m % sc_rows of the
// bf16 buffer sc_dst[m / sc_rows] (ld = ldc), which may be a peer GPU's memory; when the whole grid
// is done, sc_epoch is stored (release, system scope) to sc_flags[q][sc_flag_index] of every
// q < sc_R.  sc_counter: zeroed device int (last-CTA detection).
struct GemmScatterParams : GemmParams {
  void* sc_dst[8];
  int* sc_flags[8];
  int sc_rows, sc_R, sc_flag_index, sc_epoch;
  unsigned int* sc_counter;
};


// All-gather half of a fused all-gather + GEMM kernel: extra warps of the GEMM pull the peers' shards of
// the unit into the local unsharded buffer with plain 16-byte peer loads, chunk by chunk, and publish a
// per-chunk flag that the TMA producers wait for (gate_* fields of GemmParams).
constexpr int AG_MAX_R = 8;
struct AgParams {
  const uint4* src[AG_MAX_R];  // shard base of every rank of the group (peer-mapped)
  uint4* dst;                  // local unsharded buffer
  long shard_bytes;
  int R, r;
  int chunk_bytes, cps;        // chunk size and chunks per shard
  int* chunk_flags;            // local, [R * cps]
  int epoch;
  const int* version_flags;    // local, [R]: peers publish the epoch of their bf16 shard here
  int need_version;
};

// Selects the 2-CTA kernel with the four all-gather copy warps per CTA.
struct GemmAgParams : GemmParams {
  AgParams ag;
};


// Selects the kernels whose accumulate epilogue (C += result, bf16) reads the old C tile before the tile's
// accumulators are ready, so that the read latency hides behind the main loop (weight gradients).
struct GemmAccPrefetchParams : GemmParams {};


__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}


struct EpilogueCfg {
  bool out_f32, accum, vec_ok;
};

__device__ __forceinline__ EpilogueCfg epilogue_cfg(const GemmParams& p) {
  EpilogueCfg e;
  e.out_f32 = (p.flags & GEMM_OUT_F32) != 0;
  e.accum = (p.flags & GEMM_ACCUMULATE) != 0;
  e.vec_ok = (p.ldc % 8 == 0) && (p.addend == nullptr || p.ld_addend % 8 == 0) &&
             ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.addend) & 15) == 0);
  return e;
}

// r: 32 consecutive accumulator columns [col0, col0+32) of output row `row` (row < M checked by the caller).
__device__ __forceinline__ void epilogue_store_chunk(const GemmParams& p, const EpilogueCfg& e, int row, int col0,
                                                     const uint32_t (&r)[32]) {
  const bool out_f32 = e.out_f32, accum = e.accum, vec_ok = e.vec_ok;
  if (!zb_in_bounds(row >= 0 && row < p.M && col0 >= 0 && col0 < p.N && p.C != nullptr, p.status, 2)) return;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        const bool full_cols = (col0 + 32 <= p.N);
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (full_cols || col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
        }
        if (p.flags & GEMM_GELU) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
        } else if (p.flags & GEMM_RELU) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.f);
        }
        if (full_cols && vec_ok) {
          if (p.addend != nullptr) {
            const uint4* ap = reinterpret_cast<const uint4*>(p.addend + size_t(row) * p.ld_addend + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 a = ap[j];
              float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z),
                     f3 = unpack_bf16x2(a.w);
              v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
              v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
            }
          }
          if (out_f32) {
            float4* cp = reinterpret_cast<float4*>(static_cast<float*>(p.C) + size_t(row) * p.ldc + col0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float4 o = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
              if (accum) {
                float4 old = cp[j];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              cp[j] = o;
            }
          } else {
            uint4* cp = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc + col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (accum) {
                uint4 a = cp[j];
                float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z),
                       f3 = unpack_bf16x2(a.w);
                v[j * 8 + 0] += f0.x; v[j * 8 + 1] += f0.y; v[j * 8 + 2] += f1.x; v[j * 8 + 3] += f1.y;
                v[j * 8 + 4] += f2.x; v[j * 8 + 5] += f2.y; v[j * 8 + 6] += f3.x; v[j * 8 + 7] += f3.y;
              }
              uint4 o;
              o.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
              o.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
              o.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
              o.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
              cp[j] = o;
            }
          }
        } else {
          for (int i = 0; i < 32; ++i) {
            const int col = col0 + i;
            if (col >= p.N) break;
            float x = v[i];
            if (p.addend != nullptr) x += __bfloat162float(p.addend[size_t(row) * p.ld_addend + col]);
            if (out_f32) {
              float* cp = static_cast<float*>(p.C) + size_t(row) * p.ldc + col;
              *cp = accum ? (*cp + x) : x;
            } else {
              __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc + col;
              *cp = __float2bfloat16(accum ? (__bfloat162float(*cp) + x) : x);
            }
          }
        }
      }

// Scatter epilogue: 32 accumulator columns [col0, col0+32) as bf16 to `crow` (the destination row,
// possibly in a peer GPU's memory); plain 16-byte stores when aligned.
__device__ __forceinline__ void epilogue_scatter_chunk(__nv_bfloat16* crow, int col0, int N, bool vec_ok,
                                                       const uint32_t (&r)[32]) {
  if (vec_ok && col0 + 32 <= N) {
    uint4* cp = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 o;
      o.x = pack_bf16x2(__uint_as_float(r[j * 8 + 0]), __uint_as_float(r[j * 8 + 1]));
      o.y = pack_bf16x2(__uint_as_float(r[j * 8 + 2]), __uint_as_float(r[j * 8 + 3]));
      o.z = pack_bf16x2(__uint_as_float(r[j * 8 + 4]), __uint_as_float(r[j * 8 + 5]));
      o.w = pack_bf16x2(__uint_as_float(r[j * 8 + 6]), __uint_as_float(r[j * 8 + 7]));
      cp[j] = o;
    }
  } else {
    for (int i = 0; i < 32; ++i) {
      if (col0 + i >= N) break;
      crow[col0 + i] = __float2bfloat16(__uint_as_float(r[i]));
    }
  }
}

}  // namespace zb
