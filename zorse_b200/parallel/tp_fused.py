"""Tensor-parallel lane whose row-split GEMMs send their reduce-scatter from inside the GEMM.

`FusedTPComm.linear_rs` replaces "GEMM, then NCCL reduce-scatter, then residual / bias adds" by
two kernels of this repository:

* the 2-CTA tcgen05 GEMM with a scatter epilogue (csrc/gemm/gemm2_bf16.cu): every output row leaves
  tensor memory straight into the staging slot of the process that owns the row, with plain
  stores over NVLink, tile by tile while the main loop works on the next tile; the last CTA raises
  one flag per owner;
* `rs_finish` (csrc/comm/tp_rs.cu) on the owner: bounded wait for the lane's flags, fp32 sum of the
  slots in rank order, residual and bias added in the same pass.

Staging memory is two buffers of [tp, rows, hidden] bf16 in symmetric memory
(`torch.distributed._symmetric_memory` only allocates and exchanges the handles), used alternately
by operation count; why that needs no second handshake is written in tp_rs.cu.  Every process of
a lane must run the same sequence of `linear_rs` calls, which holds because they run the same
schedule on the same microbatches.

Opt-in (`ZORSE_TP_FUSED=1`, CUDA with the sm100 ops): built and reviewed, not yet run on a GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.tp_layers import TPComm


class FusedTPComm(TPComm):
    def __init__(self, pg, size: int, index: int, *, device: torch.device, rows: int, hidden: int, kernels):
        super().__init__(pg, size, index)
        import torch.distributed._symmetric_memory as symm

        if size > 8:
            raise ValueError("the scatter GEMM addresses at most 8 processes")
        self.k, self.device, self.n_rows, self.hidden = kernels, device, rows, hidden
        self.slot = rows * hidden                     # elements of one sender's slot
        self.stage = symm.empty(2 * size * self.slot, dtype=torch.bfloat16, device=device)
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.stage.zero_()
        self.flags.zero_()
        torch.cuda.synchronize()
        h_stage, h_flags = symm.rendezvous(self.stage, pg), symm.rendezvous(self.flags, pg)
        self._handles = (h_stage, h_flags)
        self.stage_ptrs = [int(h_stage.buffer_ptrs[q]) for q in range(size)]
        self.flag_ptrs = [int(h_flags.buffer_ptrs[q]) for q in range(size)]
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.n_ops = 0
        dist.barrier(group=pg)

    def linear_rs(self, ops, x, w, w_kmajor: bool, resid=None, bias=None):
        T = x.shape[0]
        N = w.shape[0] if w_kmajor else w.shape[1]
        if T != self.n_rows * self.size or N != self.hidden or T < 256 or N < 256:
            return super().linear_rs(ops, x, w, w_kmajor, resid, bias)      # the same choice on every process
        i = self.n_ops
        self.n_ops += 1
        par, epoch, R, r = i & 1, i + 1, self.size, self.index
        mine = (par * R + r) * self.slot * 2       # byte offset of this sender's slot in an owner's buffer
        self.k.gemm_rs(x, w, b_mn=not w_kmajor, dst_ptrs=[p + mine for p in self.stage_ptrs],
                       flag_ptrs=self.flag_ptrs, flag_index=par * R + r, epoch=epoch, counter=self.counter,
                       ldc=self.hidden)
        out = torch.empty(self.n_rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        slots = self.stage[par * R * self.slot:(par + 1) * R * self.slot]
        return self.k.rs_finish(slots, self.flags[par * R:(par + 1) * R], R, self.n_rows, self.hidden, epoch, out,
                                resid=resid, bias=bias)
