// Shared by the attention backward kernels: launch parameters and the two small helper passes
// (delta = rowsum(dO * O) before, fp32 dQ accumulator -> bf16 after).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace zb {

struct AttnBwdParams {
  const float* lse;
  const float* delta;
  float* dq_acc;          // [B*S, Hq*D] fp32, zero on entry
  __nv_bfloat16* dqkv;    // [B*S, (Hq+2Hkv)*D]
  int B, S, Hq, Hkv;
  int window, causal;
  float scale, scale_log2;
  int* status;
};

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]
int attn_bwd_delta(const __nv_bfloat16* o, const __nv_bfloat16* d_o, float* delta, int B, int S, int Hq, int D,
                   cudaStream_t stream);
// dqkv[:, :Hq*D] = bf16(dq_acc); dq_acc is left zeroed for the next call
int attn_bwd_finish_dq(float* dq_acc, __nv_bfloat16* dqkv, int B, int S, int Hq, int Hkv, int D, cudaStream_t stream);

}  // namespace zb
