"""Tensor-parallel lane whose collectives are done by the kernels that produce and consume the rows.

Reduce-scatter half.  `FusedTPComm.linear_rs` replaces "GEMM, then NCCL reduce-scatter, then residual /
bias adds" by two kernels of this repository:

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

All-gather half.  `norm_gather` / `linear_rs_norm_gather` run one row-per-CTA kernel that (sums the
slots, adds residual and bias,) normalises this process's rows and stores them into every lane member's
gathered [tokens, hidden] buffer; `gather_rows` does the same for rows that need no arithmetic.  The
consumer GEMM follows a bounded wait on the lane's flags and reads its own gathered buffer.  Two gathered
buffers alternate: a process pushes gather i + 2 only after its wait of gather i + 1 returned, that is after
every peer pushed i + 1, which each peer does after the GEMMs that read its buffer of gather i.

Opt-in (`ZORSE_TP_FUSED=1`, CUDA with the sm100 ops): built and reviewed, protocol tested with stand-in
kernels on threads, not yet run on a GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.tp_layers import TPComm


def symmetric_buffers(pg, size: int, device: torch.device, stage_elems: int):
    """Staging buffer and flag words in symmetric memory: (stage, flags, every process's stage address,
    every process's flag address)."""
    import torch.distributed._symmetric_memory as symm

    stage = symm.empty(stage_elems, dtype=torch.bfloat16, device=device)
    flags = symm.empty(64, dtype=torch.int32, device=device)
    stage.zero_()
    flags.zero_()
    torch.cuda.synchronize()
    h_stage, h_flags = symm.rendezvous(stage, pg), symm.rendezvous(flags, pg)
    dist.barrier(group=pg)
    stage._zb_handle, flags._zb_handle = h_stage, h_flags      # keep the mappings alive with the tensors
    return (stage, flags, [int(h_stage.buffer_ptrs[q]) for q in range(size)],
            [int(h_flags.buffer_ptrs[q]) for q in range(size)])


class FusedTPComm(TPComm):
    def __init__(self, pg, size: int, index: int, *, device: torch.device, rows: int, hidden: int, kernels,
                 buffers=symmetric_buffers):
        super().__init__(pg, size, index)
        if size > 8:
            raise ValueError("the scatter GEMM addresses at most 8 processes")
        if 2 * size > 64:
            raise ValueError("flag block too small")
        self.k, self.device, self.n_rows, self.hidden = kernels, device, rows, hidden
        self.slot = rows * hidden                     # elements of one sender's slot
        # one symmetric allocation: two reduce-scatter staging buffers [size][rows][hidden], then two gathered
        # buffers [size * rows][hidden]; flag words [0, 2 size) belong to the former, [16, 16 + 2 size) to the latter
        half = 2 * size * self.slot
        self.stage, self.flags, self.stage_ptrs, self.flag_ptrs = buffers(pg, size, device, 2 * half)
        self.gather_off = half                        # element offset of the gathered buffers
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.counter_g = torch.zeros(1, dtype=torch.int32, device=device)
        self.n_ops = 0
        self.n_gathers = 0

    def linear_rs(self, ops, x, w, w_kmajor: bool, resid=None, bias=None):
        T = x.shape[0]
        N = w.shape[0] if w_kmajor else w.shape[1]
        if T != self.n_rows * self.size or N != self.hidden or T < 256 or N < 256:
            return super().linear_rs(ops, x, w, w_kmajor, resid, bias)      # the same choice on every process
        return self.finish(self.send(x, w, w_kmajor), resid, bias)

    def send(self, x, w, w_kmajor: bool) -> tuple[int, int]:
        """Scatter GEMM of this process's partial product; returns (buffer parity, epoch) of the operation."""
        i = self.n_ops
        self.n_ops += 1
        par, epoch, R, r = i & 1, i + 1, self.size, self.index
        mine = (par * R + r) * self.slot * 2       # byte offset of this sender's slot in an owner's buffer
        self.k.gemm_rs(x, w, b_mn=not w_kmajor, dst_ptrs=[p + mine for p in self.stage_ptrs],
                       flag_ptrs=self.flag_ptrs, flag_index=par * R + r, epoch=epoch, counter=self.counter,
                       ldc=self.hidden)
        return par, epoch

    def finish(self, op: tuple[int, int], resid=None, bias=None) -> torch.Tensor:
        """Sum of the lane's slots for this process's rows (+ residual, + bias) once every sender's flag is up."""
        par, epoch = op
        R = self.size
        out = torch.empty(self.n_rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        slots = self.stage[par * R * self.slot:(par + 1) * R * self.slot]
        return self.k.rs_finish(slots, self.flags[par * R:(par + 1) * R], R, self.n_rows, self.hidden, epoch, out,
                                resid=resid, bias=bias)

    # ---- all-gather half: producers push rows into every lane member's gathered buffer ------------------
    GATHER_FLAGS = 16

    def _next_gather(self):
        """(parity, epoch, destinations of this process's row block, flag index) of the next gather."""
        i = self.n_gathers
        self.n_gathers += 1
        par, R, r = i & 1, self.size, self.index
        off = (self.gather_off + par * R * self.slot + r * self.slot) * 2
        return par, i + 1, [p + off for p in self.stage_ptrs], self.GATHER_FLAGS + par * R + r

    def _gathered(self, par: int, epoch: int) -> torch.Tensor:
        """This process's gathered buffer of `par` once every lane member's flag has reached `epoch`."""
        R = self.size
        self.k.wait_flags(self.flags[self.GATHER_FLAGS:], R, par, epoch)
        a = self.gather_off + par * R * self.slot
        return self.stage[a:a + R * self.slot].view(R * self.n_rows, self.hidden)

    def _fits(self, x) -> bool:
        return (x.dim() == 2 and tuple(x.shape) == (self.n_rows, self.hidden) and x.dtype == torch.bfloat16
                and x.is_contiguous())

    def gather_rows(self, x):
        if not self._fits(x):
            return super().gather_rows(x)
        par, epoch, dst, fi = self._next_gather()
        self.k.tp_push(x, dst, self.flag_ptrs, fi, epoch, self.counter_g)
        return self._gathered(par, epoch)

    def norm_gather(self, ops, x, w, b, eps, kind):
        if not self._fits(x):
            return super().norm_gather(ops, x, w, b, eps, kind)
        par, epoch, dst, fi = self._next_gather()
        n = torch.empty_like(x)
        st = torch.empty(self.n_rows, 2, dtype=torch.float32, device=self.device)
        self.k.tp_norm_push(x=x, w=w, b=b if kind == "ln" else None, eps=eps, layernorm=kind == "ln", y_local=n,
                            dst_ptrs=dst, flag_ptrs=self.flag_ptrs, flag_index=fi, epoch=epoch, stats=st,
                            counter=self.counter_g)
        return n, st, self._gathered(par, epoch)

    def linear_rs_norm_gather(self, ops, x, wmat, w_kmajor, resid, bias, w, b, eps, kind):
        T = x.shape[0]
        N = wmat.shape[0] if w_kmajor else wmat.shape[1]
        if T != self.n_rows * self.size or N != self.hidden or T < 256 or N < 256:
            return super().linear_rs_norm_gather(ops, x, wmat, w_kmajor, resid, bias, w, b, eps, kind)
        rs_par, rs_epoch = self.send(x, wmat, w_kmajor)
        par, epoch, dst, fi = self._next_gather()
        R = self.size
        h = torch.empty(self.n_rows, self.hidden, dtype=torch.bfloat16, device=self.device)
        n = torch.empty_like(h)
        st = torch.empty(self.n_rows, 2, dtype=torch.float32, device=self.device)
        slots = self.stage[rs_par * R * self.slot:(rs_par + 1) * R * self.slot]
        self.k.tp_norm_push(slots=slots, in_flags=self.flags[rs_par * R:(rs_par + 1) * R], in_epoch=rs_epoch, resid=resid,
                            bias=bias, h_out=h, w=w, b=b if kind == "ln" else None, eps=eps, layernorm=kind == "ln",
                            y_local=n, dst_ptrs=dst, flag_ptrs=self.flag_ptrs, flag_index=fi, epoch=epoch, stats=st,
                            counter=self.counter_g)
        return h, n, st, self._gathered(par, epoch)
