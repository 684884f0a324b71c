"""ZeRO unit whose two collectives run inside this repository's own kernels over NVLink.

`collectives="fused"` (CUDA, shard group of 2..8 GPUs on one NVSwitch domain):

* the unit's unsharded bf16 parameter buffer and its gradient bucket live in symmetric
  memory (`torch.distributed._symmetric_memory` is only the allocator and the handle
  exchange; the protocol is in the kernels), so every rank can address its peers' copies;
* **all-gather + GEMM**: the first GEMM that consumes the unit after a parameter update
  (QKV projection of a block, vocabulary projection of the head) is launched as
  `ag_gemm`: extra warps of the same kernel pull the peers' shards with plain peer loads,
  chunk by chunk, while tensor-core tiles whose weight rows are already present run;
* **reduce-scatter + Adam**: `rs_adam` sums this rank's slice of all R buckets with peer
  loads, applies Adam to the fp32 master shard and rewrites the bf16 shard in place inside
  the unsharded buffer — hence this mode always steps the optimizer inside backward.

Cross-GPU ordering is by epoch flags in symmetric memory (see csrc/comm/rs_adam.cu); every
device-side wait is bounded and reports through the kernel status word.  The unsharded
buffer is persistent (parameter memory as in ZeRO-2), gradients and optimizer state stay
sharded.  Replaces the NCCL calls at reference utils/patch.py:500-501, 585-589.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.layers import Layer
from ..utils import canary
from ..utils.ranges import phase
from .zero import ZeroUnit

# Granularity at which gathered weight rows become visible to the GEMM tiles waiting for them: every CTA copies one
# chunk at a time.  256 KiB is the size the multi-GPU tests and measurements ran with; smaller chunks (a multiple of
# 2 KiB, e.g. ZORSE_AG_CHUNK_BYTES=32768) let the first tiles start earlier at the price of more flag traffic.
CHUNK_BYTES = int(os.environ.get("ZORSE_AG_CHUNK_BYTES", str(1 << 18)))
# candidates of the reduce-scatter + Adam kernel that use NVSwitch multicast (csrc/comm/rs_adam.cu):
# 2 = gradient slice summed inside the switch; 3 = as 2, and the refreshed bf16 shard is stored through
# the multicast address of the unsharded buffers, so that no all-gather follows an update at all
RS_ADAM_MODE = int(os.environ.get("ZORSE_RS_ADAM_VARIANT", "1"))


@dataclass
class GatherInfo:
    """What the first GEMM of a unit needs to pull the peers' shards while it runs."""
    full: torch.Tensor
    layout: dict
    shard_ptrs: list
    R: int
    r: int
    shard_n: int
    chunk_bytes: int
    chunk_flags: torch.Tensor
    epoch: int
    version_flags: torch.Tensor
    need_version: int


class FusedZeroUnit(ZeroUnit):
    def __init__(self, layer: Layer, gid: int, **kw):
        super().__init__(layer, gid, **kw)
        if not self.cuda or self.R < 2:
            raise ValueError("fused collectives need CUDA and a shard group of at least 2 ranks")
        if self.rep_group.size > 1:
            raise NotImplementedError("fused collectives do not cover hybrid (shard x replicate) groups")
        if self.cfg.offload_params:
            raise NotImplementedError("fused collectives keep parameters on the device (no offload)")
        if self.cfg.compute_dtype != torch.bfloat16:
            raise ValueError("fused collectives need bfloat16 parameters")
        import torch.distributed._symmetric_memory as symm

        pg = self.shard_group.pg
        dev = self.device
        R, r, n, sn = self.R, self.r, self.n, self.shard_n
        # debug (ZORSE_DEBUG_CANARY=1): guard bands around the peer-visible buffers; every rank shifts
        # its payload by the same number of bytes inside the symmetric allocation
        guard = canary.enabled()
        gd = lambda dt: canary.guard_elems(dt) if guard else 0
        raw_full = symm.empty(n + 2 * gd(torch.bfloat16), dtype=torch.bfloat16, device=dev)
        raw_grad = symm.empty(n + 2 * gd(self.cfg.reduce_dtype), dtype=self.cfg.reduce_dtype, device=dev)
        raw_flag = symm.empty(64 + 2 * gd(torch.int32), dtype=torch.int32, device=dev)
        if guard:
            self.full_sym = canary.register(f"unit {gid} parameters (rank {self.rank})", raw_full, n)
            self.grad_sym = canary.register(f"unit {gid} gradients (rank {self.rank})", raw_grad, n)
            self.flags_sym = canary.register(f"unit {gid} flags (rank {self.rank})", raw_flag, 64)
        else:
            self.full_sym, self.grad_sym, self.flags_sym = raw_full, raw_grad, raw_flag
        off_full = gd(torch.bfloat16) * 2
        off_grad = gd(self.cfg.reduce_dtype) * raw_grad.element_size()
        off_flag = gd(torch.int32) * 4
        self.full_sym.zero_()
        self.grad_sym.zero_()
        self.flags_sym.zero_()
        self.full_sym[r * sn:(r + 1) * sn].copy_(self.p_shard)
        torch.cuda.synchronize()
        h_full = symm.rendezvous(raw_full, pg)
        h_grad = symm.rendezvous(raw_grad, pg)
        h_flag = symm.rendezvous(raw_flag, pg)
        self.shard_ptrs = [int(h_full.buffer_ptrs[q]) + off_full + q * sn * 2 for q in range(R)]
        self.grad_ptrs = [int(h_grad.buffer_ptrs[q]) + off_grad for q in range(R)]
        self.flag_ptrs = [int(h_flag.buffer_ptrs[q]) + off_flag for q in range(R)]
        self._handles = (h_full, h_grad, h_flag)
        self.grad_mc = self.shard_mc = 0
        self.pushed_version = -1      # update whose shards the peers stored into this rank's buffer
        if RS_ADAM_MODE in (2, 3):
            mc_g = int(getattr(h_grad, "multicast_ptr", 0) or 0)
            mc_f = int(getattr(h_full, "multicast_ptr", 0) or 0)
            if mc_g == 0 or mc_f == 0:
                raise RuntimeError("ZORSE_RS_ADAM_VARIANT=2/3 needs NVLS multicast, which this group's symmetric "
                                   "memory does not provide")
            self.grad_mc = mc_g + off_grad
            if RS_ADAM_MODE == 3:
                self.shard_mc = mc_f + off_full + r * sn * 2
        self.p_shard = self.full_sym[r * sn:(r + 1) * sn]
        self.full = self.full_sym
        self.cps = (sn * 2 + CHUNK_BYTES - 1) // CHUNK_BYTES
        self.chunk_flags = torch.zeros(R * self.cps, dtype=torch.int32, device=dev)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.version_flags = self.flags_sym[2 * R:3 * R]
        self.updates = 0          # optimizer updates done = version the shards must have
        self.gathered_version = -1
        self.gather_epoch = 0
        lay, _ = layer.layout()
        self.first_gemm = next((nm for nm in ("qkv_w", "head_w") if nm in lay), None)
        dist.barrier(group=pg)

    # ------------------------------------------------------------------ parameters
    def prefetch(self):
        return  # the gather rides on the unit's first GEMM

    def acquire(self) -> None:
        cur = torch.cuda.current_stream()
        if self.update_event is not None:
            cur.wait_event(self.update_event)
        self.layer.bind(self.full_sym, self.grad)
        if self.gathered_version == self.updates:
            return
        k = self.ops.k
        if self.pushed_version == self.updates:
            # every owner stored its refreshed shard into this rank's buffer from inside its optimizer
            # kernel; what is left of the all-gather is the wait for their version flags
            k.wait_flags(self.flags_sym, self.R, 2, self.updates)
            self.gathered_version = self.updates
            return
        self.gather_epoch += 1
        self.counters.all_gathers += 1
        lay, _ = self.layer.layout()
        if self.first_gemm is None:
            # no GEMM consumer (embedding tables): gather the whole unit with the pull kernel
            k.wait_flags(self.flags_sym, self.R, 2, self.updates)
            for q in range(self.R):
                if q != self.r:
                    k.peer_pull(self.shard_ptrs[q], self.full_sym[q * self.shard_n:], self.shard_n * 2)
        else:
            lead = lay[self.first_gemm][0]
            if lead > 0 and self.r != 0:
                # small leading parameters (norm weights) are needed before the GEMM starts
                k.wait_flags(self.flags_sym, self.R, 2, self.updates)
                k.peer_pull(self.shard_ptrs[0], self.full_sym, min(lead, self.shard_n) * 2)
            self.layer._ag = GatherInfo(self.full_sym, lay, self.shard_ptrs, self.R, self.r, self.shard_n, CHUNK_BYTES,
                                        self.chunk_flags, self.gather_epoch, self.version_flags, self.updates)
        self.gathered_version = self.updates

    def release(self, force: bool = False) -> None:
        return

    # ------------------------------------------------------------------ gradients
    def grad_views(self) -> None:
        if self.grad is None:
            if self.update_event is not None:
                torch.cuda.current_stream().wait_event(self.update_event)
            self.grad = self.grad_sym
        self.layer.bind(self.full_sym, self.grad)

    def reduce_grads(self) -> None:
        if self.grad is None:
            self.grad = self.grad_sym  # a rank without microbatches still takes part
        self.grad = None
        self.layer.bind(self.full_sym, None)
        a = self.cfg.adam
        self.step_count += 1
        self.updates += 1
        gscale = 1.0 / self.R if self.cfg.grad_divide_by_group else 1.0
        k = self.ops.k
        cur = torch.cuda.current_stream()
        self.streams.comm.wait_stream(cur)
        with phase("zero.rs_adam_fused"), torch.cuda.stream(self.streams.comm):
            kw = dict(lr=a.lr, beta1=a.beta1, beta2=a.beta2, eps=a.eps, weight_decay=a.weight_decay,
                      step=self.step_count, grad_scale=gscale, grad_f32=self.cfg.reduce_dtype == torch.float32,
                      epoch=self.updates, counter=self.counter)
            if self.grad_mc:
                k.rs_adam_nvls(self.grad_mc, self.flag_ptrs, self.R, self.r, self.shard_n, self.master, self.m,
                               self.v, self.p_shard, p16_mc=self.shard_mc, **kw)
                if self.shard_mc:
                    self.pushed_version = self.updates
            else:
                k.rs_adam(self.grad_ptrs, self.flag_ptrs, self.R, self.r, self.shard_n, self.master, self.m, self.v,
                          self.p_shard, **kw)
            # the bucket may be cleared once every peer has read its slice of it
            k.wait_flags(self.flags_sym, self.R, 1, self.updates)
            self.grad_sym.zero_()
            ev = torch.cuda.Event()
            ev.record(self.streams.comm)
        self.update_event = ev
        self.counters.reduce_scatters += 1
        self.counters.adam_steps += 1

    def optimizer_step(self) -> None:
        return

    def finish_step(self) -> None:
        return

    def _after_update(self):
        self.full_sym[self.r * self.shard_n:(self.r + 1) * self.shard_n].copy_(self.master.to(torch.bfloat16))
        dist.barrier(group=self.shard_group.pg)
        self.gathered_version = self.pushed_version = -1
