// Receive half of the row-wise reduce-scatter that is fused into a tensor-parallel GEMM.
//
// The row-split GEMMs of a tensor-parallel lane (attention output, MLP down projection, and the
// input gradients of the column-split ones) produce partial sums of a [T, H] tensor on each of the
// R processes, and every process needs the sum of its own T/R rows.  The scatter GEMM
// (gemm2_bf16_kernel<.., SCATTER>) stores each row, as it leaves tensor memory, into the owner's
// staging buffer slot [sender][row][H] with plain stores over NVLink, and raises one flag per
// sender when its grid is done.  This kernel is the owner's side: it waits (bounded) for the R
// flags, adds the R slots in fp32 in rank order (deterministic), adds the residual rows and the
// bias if given, and writes bf16.
//
// Staging buffers are used alternately by operation count (parity), which makes reuse safe without
// a second handshake: a process reaches operation i + 2 only after its own finish of operation
// i + 1, which needed every peer's scatter GEMM of i + 1, which follows the peer's finish of
// operation i in stream order.  (Replaces the NCCL reduce_scatter_tensor of the library path; the
// reference has tensor parallelism only as an unused plan, models/parallelize_model.py:107-173.)
#include "../common/host.h"
#include "../common/ptx.cuh"

namespace zb {

struct RsFinishParams {
  const __nv_bfloat16* slots;   // [R][rows][ld] bf16, this process's staging buffer of the parity in use
  const int* flags;             // R ints: epoch of the last complete scatter of every sender
  const __nv_bfloat16* resid;   // [rows][ld_resid] or nullptr
  const __nv_bfloat16* bias;    // [H] or nullptr
  __nv_bfloat16* out;           // [rows][ld_out]
  int R, rows, H, ld, ld_resid, ld_out, epoch;
  unsigned long long wait_ns;
  int* status;
};

__global__ void __launch_bounds__(256)
rs_finish_kernel(const RsFinishParams p) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    bool ok = true;
    for (int q = 0; q < p.R && ok; ++q) ok = flag_wait_ge(p.flags + q, p.epoch, p.wait_ns, p.status, ST_TIMEOUT_FLAG);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const int vec_per_row = p.H >> 3;
  const long nvec = long(p.rows) * vec_per_row;
  const size_t slot_stride = size_t(p.rows) * p.ld;
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < nvec; i += long(gridDim.x) * blockDim.x) {
    const int row = int(i / vec_per_row), c = int(i % vec_per_row) * 8;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int q = 0; q < p.R; ++q) {
      // the slots were written by other GPUs: read them past any stale cached line
      const uint4 u = ld_v4_relaxed_sys(p.slots + q * slot_stride + size_t(row) * p.ld + c);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), d = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += d.x; acc[5] += d.y; acc[6] += e.x; acc[7] += e.y;
    }
    if (p.resid != nullptr) {
      const uint4 u = *reinterpret_cast<const uint4*>(p.resid + size_t(row) * p.ld_resid + c);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), d = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += d.x; acc[5] += d.y; acc[6] += e.x; acc[7] += e.y;
    }
    if (p.bias != nullptr) {
      const uint4 u = *reinterpret_cast<const uint4*>(p.bias + c);
      const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), d = unpack_bf16x2(u.z), e = unpack_bf16x2(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += d.x; acc[5] += d.y; acc[6] += e.x; acc[7] += e.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(p.out + size_t(row) * p.ld_out + c) = o;
  }
}

}  // namespace zb

extern "C" int zb_rs_finish(const void* slots, const int* flags, int R, int rows, int H, int ld, int epoch,
                            const void* resid, int ld_resid, const void* bias, void* out, int ld_out,
                            double wait_seconds, int* status, cudaStream_t stream) {
  using namespace zb;
  if (R < 1 || R > 8) ZB_FAIL(-1, "rs_finish: group size %d unsupported (1..8)", R);
  if (rows <= 0 || H <= 0) return 0;
  if (H % 8 || ld % 8 || ld_out % 8 || (resid != nullptr && ld_resid % 8))
    ZB_FAIL(-1, "rs_finish: widths and row strides must be multiples of 8 elements");
  if ((reinterpret_cast<uintptr_t>(slots) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(resid) |
       reinterpret_cast<uintptr_t>(bias)) & 15)
    ZB_FAIL(-1, "rs_finish: pointers must be 16-byte aligned");
  RsFinishParams p;
  p.slots = static_cast<const __nv_bfloat16*>(slots);
  p.flags = flags;
  p.resid = static_cast<const __nv_bfloat16*>(resid);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.R = R; p.rows = rows; p.H = H; p.ld = ld; p.ld_resid = ld_resid; p.ld_out = ld_out; p.epoch = epoch;
  p.wait_ns = (unsigned long long)(wait_seconds * 1e9);
  p.status = status;
  const long nvec = long(rows) * (H / 8);
  long blocks = (nvec + 255) / 256;
  const long cap = long(num_sms()) * 4;
  if (blocks > cap) blocks = cap;
  rs_finish_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

// ---------------------------------------------------------------------------------------------
// All-gather half: rows are pushed into every lane member's gathered buffer by the kernel that
// produces them.
//
// tp_norm_kernel: one CTA per row.  Input row = x[row] (SLOTS = false) or the fp32 sum of the R
// reduce-scatter slots (+ residual, + bias), rounded to bf16 and written to h_out (SLOTS = true:
// the owner side of the scatter GEMM and the normalisation behind it in one pass).  The row is
// normalised (RMSNorm or LayerNorm, statistics from the bf16 values, as the separate kernels do)
// and stored to y_local and to ndst destinations: this process's row block inside every lane
// member's gathered [T, H] buffer (plain stores over NVLink).  The last CTA raises the arrival
// flag at every destination; the consumer (a GEMM on its own gathered buffer) is preceded by a
// bounded wait on those flags.  tp_push_kernel does the same for rows that need no arithmetic
// (gradient gathers in the backward pass).  Gathered buffers alternate by operation count like the
// reduce-scatter staging buffers; between two uses of one buffer there is always a reduce-scatter
// that every lane member has to finish first.
namespace zb {

struct TpNormParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* slots;
  const int* in_flags;
  const __nv_bfloat16* resid;
  const __nv_bfloat16* bias;
  __nv_bfloat16* h_out;
  const __nv_bfloat16* w;
  const __nv_bfloat16* b;
  __nv_bfloat16* y_local;
  __nv_bfloat16* y_dst[8];
  int* out_flags[8];
  float* stats;
  unsigned int* counter;
  int* status;
  unsigned long long wait_ns;
  float eps;
  int R_in, in_epoch, ndst, out_flag_index, out_epoch, rows, H, ld_resid;
};

constexpr int TPN_THREADS = 256;
constexpr int TPN_MAXV = 4;   // H <= 8192

__device__ __forceinline__ float tpn_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (l == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ void tpn_unpack8(const uint4& u, float* f) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 tpn_pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// every thread has stored and fenced its part; the last CTA of the grid raises the flags
__device__ __forceinline__ void tp_signal_when_grid_done(unsigned int* counter, int* const* flags, int nflags,
                                                         int index, int epoch, const int* status) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(counter, 1u) == gridDim.x - 1) {
      __threadfence_system();
      if (*reinterpret_cast<const volatile int*>(status) == 0)
        for (int q = 0; q < nflags; ++q) st_release_sys(flags[q] + index, epoch);
      *counter = 0u;
    }
  }
}

template <bool LN, bool SLOTS>
__global__ void __launch_bounds__(TPN_THREADS)
tp_norm_kernel(const TpNormParams p) {
  __shared__ float red[33];
  __shared__ int s_ok;
  const int row = blockIdx.x;
  const int nchunk = p.H >> 3;
  if (SLOTS) {
    if (threadIdx.x == 0) {
      bool ok = true;
      for (int q = 0; q < p.R_in && ok; ++q)
        ok = flag_wait_ge(p.in_flags + q, p.in_epoch, p.wait_ns, p.status, ST_TIMEOUT_FLAG);
      s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!s_ok) return;     // uniform: no flag is raised, the consumers' waits report as well
  }
  float v[TPN_MAXV][8];
  float s = 0.f, ss = 0.f;
  const size_t slot_stride = size_t(p.rows) * p.H;
#pragma unroll
  for (int i = 0; i < TPN_MAXV; ++i) {
    const int c = threadIdx.x + i * TPN_THREADS;
    if (c < nchunk) {
      if (SLOTS) {
        float acc[8], t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int q = 0; q < p.R_in; ++q) {
          tpn_unpack8(ld_v4_relaxed_sys(p.slots + q * slot_stride + size_t(row) * p.H + c * 8), t);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += t[j];
        }
        if (p.resid != nullptr) {
          tpn_unpack8(*reinterpret_cast<const uint4*>(p.resid + size_t(row) * p.ld_resid + c * 8), t);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += t[j];
        }
        if (p.bias != nullptr) {
          tpn_unpack8(*reinterpret_cast<const uint4*>(p.bias + c * 8), t);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += t[j];
        }
        const uint4 h = tpn_pack8(acc);
        *reinterpret_cast<uint4*>(p.h_out + size_t(row) * p.H + c * 8) = h;
        tpn_unpack8(h, v[i]);      // statistics from the rounded values, like a separate norm kernel
      } else {
        tpn_unpack8(*reinterpret_cast<const uint4*>(p.x + size_t(row) * p.H + c * 8), v[i]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { s += v[i][j]; ss += v[i][j] * v[i][j]; }
    }
  }
  float mean = 0.f;
  if (LN) {
    mean = tpn_block_sum(s, red) / p.H;
    float d2 = 0.f;
#pragma unroll
    for (int i = 0; i < TPN_MAXV; ++i) {
      const int c = threadIdx.x + i * TPN_THREADS;
      if (c < nchunk) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { const float d = v[i][j] - mean; d2 += d * d; }
      }
    }
    ss = d2;
  }
  const float rstd = rsqrtf(tpn_block_sum(ss, red) / p.H + p.eps);
  if (threadIdx.x == 0 && p.stats != nullptr) {
    p.stats[2 * row] = mean;
    p.stats[2 * row + 1] = rstd;
  }
#pragma unroll
  for (int i = 0; i < TPN_MAXV; ++i) {
    const int c = threadIdx.x + i * TPN_THREADS;
    if (c < nchunk) {
      float wf[8], bf[8], o[8];
      tpn_unpack8(*reinterpret_cast<const uint4*>(p.w + c * 8), wf);
      if (LN && p.b != nullptr) tpn_unpack8(*reinterpret_cast<const uint4*>(p.b + c * 8), bf);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j] = (v[i][j] - mean) * rstd * wf[j];
        if (LN && p.b != nullptr) o[j] += bf[j];
      }
      const uint4 u = tpn_pack8(o);
      const size_t off = size_t(row) * p.H + c * 8;
      *reinterpret_cast<uint4*>(p.y_local + off) = u;
      for (int q = 0; q < p.ndst; ++q) *reinterpret_cast<uint4*>(p.y_dst[q] + off) = u;
    }
  }
  tp_signal_when_grid_done(p.counter, p.out_flags, p.ndst, p.out_flag_index, p.out_epoch, p.status);
}

struct TpPushParams {
  const uint4* src;
  uint4* dst[8];
  int* out_flags[8];
  unsigned int* counter;
  int* status;
  long n16;
  int ndst, out_flag_index, out_epoch;
};

__global__ void __launch_bounds__(256)
tp_push_kernel(const TpPushParams p) {
  for (long i = blockIdx.x * long(blockDim.x) + threadIdx.x; i < p.n16; i += long(gridDim.x) * blockDim.x) {
    const uint4 u = p.src[i];
    for (int q = 0; q < p.ndst; ++q) p.dst[q][i] = u;
  }
  tp_signal_when_grid_done(p.counter, p.out_flags, p.ndst, p.out_flag_index, p.out_epoch, p.status);
}

}  // namespace zb

extern "C" {

// Normalises `rows` rows of width H and stores them to y_local and to dst_ptrs[0..ndst) (this process's
// row block inside every lane member's gathered buffer); afterwards `out_epoch` is stored to
// out_flag_ptrs[q][out_flag_index].  Input: x (slots == nullptr), or the sum of the R_in reduce-scatter
// slots [R_in][rows][H] (+ resid + bias) once in_flags[0..R_in) have reached in_epoch; that sum is
// written to h_out.  counter: zeroed device int.
int zb_tp_norm_push(const void* x, const void* slots, const int* in_flags, int R_in, int in_epoch, const void* resid,
                    int ld_resid, const void* bias, void* h_out, const void* w, const void* b, float eps, int layernorm,
                    void* y_local, void* const* dst_ptrs, int* const* out_flag_ptrs, int ndst, int out_flag_index,
                    int out_epoch, float* stats, int rows, int H, unsigned int* counter, double wait_seconds,
                    int* status, cudaStream_t stream) {
  using namespace zb;
  if (rows <= 0) return 0;
  if (H % 8 != 0 || H > TPN_THREADS * TPN_MAXV * 8) ZB_FAIL(-1, "tp_norm_push: H=%d unsupported", H);
  if (ndst < 0 || ndst > 8 || R_in < 0 || R_in > 8) ZB_FAIL(-1, "tp_norm_push: at most 8 lane members");
  if ((x == nullptr) == (slots == nullptr)) ZB_FAIL(-1, "tp_norm_push: give either x or slots");
  if (slots != nullptr && (h_out == nullptr || in_flags == nullptr)) ZB_FAIL(-1, "tp_norm_push: slots need h_out and flags");
  if (resid != nullptr && ld_resid % 8) ZB_FAIL(-1, "tp_norm_push: residual stride must be a multiple of 8");
  TpNormParams p;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.slots = static_cast<const __nv_bfloat16*>(slots);
  p.in_flags = in_flags;
  p.resid = static_cast<const __nv_bfloat16*>(resid);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.h_out = static_cast<__nv_bfloat16*>(h_out);
  p.w = static_cast<const __nv_bfloat16*>(w);
  p.b = static_cast<const __nv_bfloat16*>(b);
  p.y_local = static_cast<__nv_bfloat16*>(y_local);
  for (int q = 0; q < 8; ++q) {
    p.y_dst[q] = q < ndst ? static_cast<__nv_bfloat16*>(dst_ptrs[q]) : nullptr;
    p.out_flags[q] = q < ndst ? out_flag_ptrs[q] : nullptr;
    if (q < ndst && (reinterpret_cast<uintptr_t>(dst_ptrs[q]) & 15)) ZB_FAIL(-1, "tp_norm_push: destination %d not 16-byte aligned", q);
  }
  p.stats = stats; p.counter = counter; p.status = status;
  p.wait_ns = (unsigned long long)(wait_seconds * 1e9);
  p.eps = eps;
  p.R_in = R_in; p.in_epoch = in_epoch; p.ndst = ndst; p.out_flag_index = out_flag_index; p.out_epoch = out_epoch;
  p.rows = rows; p.H = H; p.ld_resid = ld_resid;
  if (slots != nullptr) {
    if (layernorm) tp_norm_kernel<true, true><<<rows, TPN_THREADS, 0, stream>>>(p);
    else tp_norm_kernel<false, true><<<rows, TPN_THREADS, 0, stream>>>(p);
  } else {
    if (layernorm) tp_norm_kernel<true, false><<<rows, TPN_THREADS, 0, stream>>>(p);
    else tp_norm_kernel<false, false><<<rows, TPN_THREADS, 0, stream>>>(p);
  }
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

// Copies `bytes` (multiple of 16) from src to dst_ptrs[0..ndst), then raises the flags as above.
int zb_tp_push(const void* src, void* const* dst_ptrs, int* const* out_flag_ptrs, int ndst, int out_flag_index,
               int out_epoch, long bytes, unsigned int* counter, int* status, cudaStream_t stream) {
  using namespace zb;
  if (bytes <= 0) return 0;
  if (ndst < 1 || ndst > 8) ZB_FAIL(-1, "tp_push: 1..8 destinations");
  if (bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15)) ZB_FAIL(-1, "tp_push: source and size must be multiples of 16 bytes");
  TpPushParams p;
  p.src = static_cast<const uint4*>(src);
  for (int q = 0; q < 8; ++q) {
    p.dst[q] = q < ndst ? static_cast<uint4*>(dst_ptrs[q]) : nullptr;
    p.out_flags[q] = q < ndst ? out_flag_ptrs[q] : nullptr;
    if (q < ndst && (reinterpret_cast<uintptr_t>(dst_ptrs[q]) & 15)) ZB_FAIL(-1, "tp_push: destination %d not 16-byte aligned", q);
  }
  p.counter = counter; p.status = status; p.n16 = bytes / 16;
  p.ndst = ndst; p.out_flag_index = out_flag_index; p.out_epoch = out_epoch;
  long blocks = (p.n16 + 255) / 256;
  const long cap = long(num_sms()) * 4;
  if (blocks > cap) blocks = cap;
  tp_push_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p);
  ZB_CUDA_OK(cudaGetLastError());
  return 0;
}

}  // extern "C"
