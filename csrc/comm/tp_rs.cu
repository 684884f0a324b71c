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
