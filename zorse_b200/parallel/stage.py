"""Run-time object of one pipeline stage on one rank, and the activation stash.

A stage owns a contiguous range of transformer blocks (plus the embedding on the first
stage and norm + head + loss on the last), one ZeRO unit per layer, the microbatches the
static plan assigns to this rank and the four transfers of each.  A rank may hold several
stages (interleaving), as in the reference (zorse_utils/pipeline.py:36-318).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..config.training_config import PipelineConfig, StageConfig
from ..engine.zero import EngineConfig, StageEngine, Streams
from ..models import registry
from .groups import StageGroups
from ..utils import canary
from ..utils import stream_check as SC
from ..utils.ranges import phase
from .p2p import LocalMailbox
from .p2p_plan import StageCommPattern, is_regular


class ActivationStash:
    """Layer-boundary activations of a stage, keyed by (layer, local microbatch); optionally
    parked in pinned host memory through a copy stream (the reference always does this,
    zorse_utils/pipeline_schedule_v2.py:66-84, 256-262; on a 180 GB GPU it is an option)."""

    def __init__(self, device: torch.device, offload: bool, copy_stream=None):
        self.device, self.offload = device, offload and device.type == "cuda"
        self.copy_stream = copy_stream
        self.store: dict = {}
        self.d2h_bytes = 0
        self.h2d_bytes = 0
        self._pool: dict = {}

    def put(self, key, t: torch.Tensor) -> None:
        if not self.offload or t.dtype == torch.long:
            self.store[key] = t
            return
        pk = (tuple(t.shape), t.dtype)
        free = self._pool.setdefault(pk, [])
        host = free.pop() if free else canary.guarded(
            t.numel(), t.dtype, lambda k, dt: torch.empty(k, dtype=dt, device="cpu", pin_memory=True),
            f"pinned activation buffer {tuple(t.shape)}").view(t.shape)
        SC.wrote(("stash_src", id(t)))
        self.copy_stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.copy_stream):
            SC.read(("stash_src", id(t)), label="D2H copy of an activation the compute stream produced")
            host.copy_(t, non_blocking=True)
            SC.wrote(("stash_host", key))
            ev = torch.cuda.Event()
            ev.record(self.copy_stream)
        t.record_stream(self.copy_stream)
        self.d2h_bytes += t.numel() * t.element_size()
        self.store[key] = (host, ev)

    def get(self, key, pop: bool = True):
        v = self.store.pop(key) if pop else self.store[key]
        if not isinstance(v, tuple):
            return v
        host, ev = v
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(ev)
            SC.read(("stash_host", key), label="H2D copy of a parked activation")
            dev = host.to(self.device, non_blocking=True)
            SC.wrote(("stash_dev", id(dev)))
            done = torch.cuda.Event()
            done.record(self.copy_stream)
        torch.cuda.current_stream().wait_event(done)
        SC.read(("stash_dev", id(dev)), label="compute on a restored activation")
        dev.record_stream(torch.cuda.current_stream())
        self.h2d_bytes += host.numel() * host.element_size()
        if pop:
            # the pinned buffer may be reused once the H2D copy has been issued on the same stream
            self._pool.setdefault((tuple(host.shape), host.dtype), []).append(host)
        return dev

    def clear(self):
        self.store.clear()


class DeferredWgrad:
    """Ops front that can hold back the weight-gradient GEMMs of a backward pass.

    The gradient a stage sends upstream depends only on the input-gradient GEMMs; the weight-gradient GEMMs
    (a third of a step's arithmetic) feed nothing but the gradient bucket.  While `active`, `linear_wgrad`
    calls are queued with their arguments (the views into the bucket they accumulate into stay valid), and
    `flush()` runs them in order, so a schedule can send the input gradient first and do the weight gradients
    while the upstream stage is already working: the chain between stages gets shorter by the weight-gradient
    time per stage.  Results are bit-identical: every bucket entry receives the same additions in the same order."""

    def __init__(self, ops):
        self._ops = ops
        self._queue: list = []
        self.active = False

    def __getattr__(self, name):
        return getattr(self._ops, name)

    def linear_wgrad(self, *a, **k):
        if self.active:
            self._queue.append((a, k))
        else:
            self._ops.linear_wgrad(*a, **k)

    def flush(self) -> None:
        q, self._queue = self._queue, []
        for a, k in q:
            self._ops.linear_wgrad(*a, **k)


class PipelineStage:
    def __init__(self, cfg: PipelineConfig, st: StageConfig, *, rank: int, device: torch.device, ops,
                 engine_cfg: EngineConfig, groups: StageGroups, streams: Streams, pattern: StageCommPattern,
                 transport, gloo_transport=None, activation_offload: bool = False, model_overrides: Optional[dict] = None,
                 local_mailbox=None, process_rank: Optional[int] = None, split_parity: Optional[bool] = None):
        # `rank` is the number the config and the p2p plan know this process by (its lane with tensor
        # parallelism); `process_rank` its rank in torch.distributed, which the groups are made of
        self.cfg, self.st, self.rank, self.device, self.ops = cfg, st, rank, device, ops
        process_rank = rank if process_rank is None else process_rank
        self.tp = None
        tp_size, tp_index = cfg.tensor_parallel_size, 0
        if tp_size > 1:
            from ..models.tp_layers import TPComm

            tp_index = groups.tp.index_of(process_rank)
            self.tp = TPComm(groups.tp.pg, tp_size, tp_index)
            self._tp_fused = (os.environ.get("ZORSE_TP_FUSED") == "1" and device.type == "cuda"
                              and getattr(ops, "name", "") == "sm100")
        self.stage_id = st.stage_id
        self.num_stages = len(cfg.stages)
        self.is_first = st.layer_partition[0] == 0
        self.spec = registry.get_spec(cfg.model_name, vocab=cfg.vocab_size, **(model_overrides or {}))
        self.is_last = st.layer_partition[1] == self.spec.layers
        self.layers = registry.build_stage_layers(self.spec, st.layer_partition[0], st.layer_partition[1],
                                                  cfg.sequence_length, tp=tp_size, tp_index=tp_index)
        gids = [registry.global_layer_index(self.spec, st.layer_partition[0], i, self.layers)
                for i in range(len(self.layers))]
        self.engine = StageEngine(self.layers, gids, device=device, cfg=engine_cfg, ops=ops, shard=groups.shard,
                                  replicate=groups.replicate, rank=process_rank, streams=streams,
                                  zero_level=st.zero_level, meta_init=False, shard_ratios=st.shard_ratio,
                                  tp_group=groups.tp)
        self.pattern = pattern
        # irregular routing (mixed widths / uneven counts): traffic of even and odd stage boundaries goes
        # through different process groups, so that a rank's receives (boundary b - 1) and sends (boundary b)
        # never share a serialised queue; regular plans keep the four groups they were measured with
        # (`split_parity=True`: asked for by a schedule that posts receives ahead, which needs the same separation)
        self.split_parity = (not is_regular(cfg)) if split_parity is None else bool(split_parity)
        self.pos = [s.stage_id for s in cfg.stages].index(st.stage_id)
        self.transport = transport
        self.gloo_transport = gloo_transport
        self.local = local_mailbox if local_mailbox is not None else LocalMailbox()
        self.microbatches = list(pattern.microbatches)  # global ids, increasing
        self.M = len(self.microbatches)
        self.B, self.S, self.hidden = cfg.microbatch_size, cfg.sequence_length, self.spec.hidden
        self.tokens = self.B * self.S
        if self.spec.family == "vit":
            self.S = self.layers[0].tokens_per_image() if self.is_first else (self.spec.image // self.spec.patch) ** 2 + 1
            self.tokens = self.B * self.S
        if self.tokens % tp_size:
            raise ValueError(f"{self.tokens} tokens per microbatch do not split over {tp_size} tensor-parallel processes")
        if self.tp is not None and self._tp_fused:
            from .tp_fused import FusedTPComm

            self.tp = FusedTPComm(groups.tp.pg, tp_size, tp_index, device=device, rows=self.tokens // tp_size,
                                  hidden=self.hidden, kernels=ops.k)
        self.act_dtype = engine_cfg.compute_dtype
        self.wgrad = DeferredWgrad(ops)      # what backward_layer hands to the layers as their ops
        self.wgrad_tail = DeferredWgrad(ops)  # weight gradients held back until the stage's last backward is done
        self.stash = ActivationStash(device, activation_offload, streams.copy)
        self.saved: dict = {}
        self.loss_sum: Optional[torch.Tensor] = None
        # gradient scale: true mean over every token of the global batch, or the reference's
        # arithmetic (per-microbatch mean, summed over local microbatches, averaged over DP ranks)
        per_mb = 1.0 / (self.B if self.spec.pool else self.tokens)
        if cfg.grad_norm_compat == "reference":
            self.loss_scale = per_mb
        else:
            self.loss_scale = per_mb / cfg.num_microbatches

    # -- helpers ----------------------------------------------------------------------
    def ctx(self, mbl: int, targets=None) -> dict:
        c = {"B": self.B, "S": self.S, "loss_scale": self.loss_scale}
        if self.tp is not None:
            c["tp"] = self.tp
        if targets is not None:
            c["targets"] = targets
        return c

    def act_shape(self):
        """Rows of a stage-boundary message: with tensor parallelism every process of a lane sends and
        receives only its own rows."""
        return (self.tokens // self.cfg.tensor_parallel_size, self.hidden)

    def boundary_transport(self, towards_next: bool):
        """Transport of the boundary to the next (or previous) stage.  With a Gloo communicator
        present (`--gloo_p2p`) and `alternate_nccl_gloo` set, boundaries between stages of equal
        width stay on NCCL and mixed-width boundaries (many-to-many routing) go through Gloo, as
        the reference's ZeRO-2 schedule does (zorse_utils/pipeline_schedule_zero2.py:230-244);
        without the option every boundary uses the Gloo communicator."""
        if self.gloo_transport is None:
            return self.transport
        if not self.cfg.alternate_nccl_gloo:
            return self.gloo_transport
        stages = self.cfg.stages
        pos = [s.stage_id for s in stages].index(self.stage_id)
        other = pos + 1 if towards_next else pos - 1
        if 0 <= other < len(stages) and len(stages[other].gpu_ranks) == len(self.st.gpu_ranks):
            return self.transport
        return self.gloo_transport

    def uses_gloo(self, towards_next: bool) -> bool:
        return self.gloo_transport is not None and self.boundary_transport(towards_next) is self.gloo_transport

    def transports(self):
        return [t for t in (self.transport, self.gloo_transport) if t is not None]

    def flush(self) -> None:
        for t in self.transports():
            t.flush()

    def _kind(self, base: str, towards_next: bool) -> str:
        if not self.split_parity:
            return base
        boundary = self.pos if towards_next else self.pos - 1
        return f"{base}{boundary & 1}"

    def recv_fwd(self, mbl: int):
        src, tag = self.pattern.fwd_recv[mbl]
        if src == self.rank:
            return self.local.recv(tag)
        with phase("p2p.recv_act"):
            return self.boundary_transport(False).recv(self.act_shape(), self.act_dtype, src, tag, self._kind("act", False))

    def send_fwd(self, mbl: int, y: torch.Tensor):
        dst, tag = self.pattern.fwd_send[mbl]
        if dst == self.rank:
            return self.local.send(y, tag)
        with phase("p2p.send_act"):
            return self.boundary_transport(True).send(y, dst, tag, self._kind("act", True))

    def recv_bwd(self, mbl: int):
        src, tag = self.pattern.bwd_recv[mbl]
        if src == self.rank:
            return self.local.recv(tag)
        with phase("p2p.recv_grad"):
            return self.boundary_transport(True).recv(self.act_shape(), self.act_dtype, src, tag, self._kind("grad", True))

    def send_bwd(self, mbl: int, dx: torch.Tensor):
        dst, tag = self.pattern.bwd_send[mbl]
        if dst == self.rank:
            return self.local.send(dx, tag)
        with phase("p2p.send_grad"):
            return self.boundary_transport(False).send(dx, dst, tag, self._kind("grad", False))

    def can_defer_wgrad(self) -> bool:
        """Deferred weight gradients keep their operands alive until the flush; the fused tensor-parallel lane
        hands out gathered operands in staging buffers that the next gather overwrites."""
        return type(self.tp).__name__ != "FusedTPComm"

    def add_loss(self, rows: torch.Tensor) -> None:
        v = rows.float().sum() * self.loss_scale
        self.loss_sum = v if self.loss_sum is None else self.loss_sum + v

    # -- one layer, one microbatch ---------------------------------------------------
    def forward_layer(self, li: int, mbl: int, x, targets, recompute: bool, want_loss: bool = True):
        """Runs layer li on microbatch mbl. With recompute only the layer input is stashed."""
        layer = self.layers[li]
        c = self.ctx(mbl, targets if layer.kind == "head" else None)
        with phase("fwd." + layer.kind):
            if recompute:
                self.stash.put((li, mbl), x)
                y = layer.forward(x, c, self.ops, None)
            else:
                sv: dict = {}
                y = layer.forward(x, c, self.ops, sv)
                self.saved[(li, mbl)] = sv
        if layer.kind == "head":
            if want_loss:
                self.add_loss(y)
            return None
        return y

    def backward_layer(self, li: int, mbl: int, dy, targets, recompute: bool, hold_wgrad: bool = False):
        """`hold_wgrad`: this layer's weight-gradient GEMMs go to the tail queue (`wgrad_tail`), which the schedule
        flushes once, after the stage's last backward."""
        layer = self.layers[li]
        c = self.ctx(mbl, targets if layer.kind == "head" else None)
        if recompute:
            x = self.stash.get((li, mbl))
            sv: dict = {}
            with phase("recompute." + layer.kind):
                layer.forward(x, c, self.ops, sv)
            if self.cfg.sync_after_recompute and self.device.type == "cuda":
                # `"skip_compute_sync": false` in the config: the host waits for the recomputed forward, which
                # lets the caching allocator reuse freed blocks sooner (fewer allocation retries when memory is
                # tight; reference zorse_utils/pipeline_schedule_v2.py:187-194)
                torch.cuda.current_stream().synchronize()
        else:
            sv = self.saved.pop((li, mbl))
        with phase("bwd." + layer.kind):
            if hold_wgrad:
                self.wgrad_tail.active = True
                return layer.backward(dy, c, self.wgrad_tail, sv)
            return layer.backward(dy, c, self.wgrad if self.wgrad.active else self.ops, sv)
