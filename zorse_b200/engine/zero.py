"""Explicit ZeRO engine: one `ZeroUnit` per layer (transformer block, embedding, head).

This replaces the reference's monkey-patched FSDP1 (utils/patch.py, utils/global_state.py)
with a small state machine per unit that the pipeline schedules drive directly:

    prefetch() / acquire()   all-gather the unit's bf16 shards into an unsharded buffer,
                             once per pass however many microbatches run  (patch.py:854-887)
    release()                drop the unsharded buffer (ZeRO-3) after the last microbatch
                             of a pass; ZeRO-2 units keep it until the step ends (:512-551, :788-795)
    grad_views()             gradient bucket in `reduce_dtype`, allocated on first use in a
                             step; backward kernels accumulate into it across microbatches (:202-219)
    reduce_grads()           after the unit's last microbatch: reduce-scatter inside the shard
                             group (+ all-reduce across replicate groups = hybrid shard), then
                             either Adam right away (optimizer-in-backward, :76-154) or
                             accumulation into a gradient shard that `optimizer_step` consumes
    offload                  fp32 master + bf16 shard parked in pinned host memory between uses,
                             copied on a dedicated copy stream (:61-73, :1159-1187)

Per shard group of size R the flat buffer is padded to a multiple of R*ALIGN elements and
rank r owns elements [r*n/R, (r+1)*n/R).  With `shard_ratios` the ranks own unequal,
ALIGN-rounded ranges instead (the reference's dormant uneven-shard path,
utils/patch.py:308-441, 470-498, 244-275): the gather becomes one broadcast per owner and
the reduce-scatter one reduce per owner, both of which every backend supports for unequal
sizes.  Collectives run on a side stream; the compute stream waits on a per-unit event,
never on the whole stream (patch.py:873-879).  On CPU (gloo) everything is synchronous.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from ..models.layers import ALIGN, Layer
from ..parallel.groups import Group
from ..utils import stream_check as SC
from ..utils.ranges import phase


def shard_bounds(n: int, R: int, ratios=None) -> list[int]:
    """Element offsets [o_0 = 0, ..., o_R = n] of the R shards of a flat buffer of n elements
    (n a multiple of R*ALIGN).  Without ratios the shards are equal; with ratios rank q gets
    about ratios[q] / sum(ratios) of the buffer, rounded to ALIGN elements, the last rank the
    remainder; every rank keeps at least one ALIGN block."""
    if ratios is None:
        return [q * (n // R) for q in range(R + 1)]
    if len(ratios) != R or any(x <= 0 for x in ratios):
        raise ValueError(f"shard_ratios needs {R} positive entries, got {list(ratios)}")
    blocks = n // ALIGN
    tot = float(sum(ratios))
    offs, acc = [0], 0.0
    for q in range(R - 1):
        acc += ratios[q] / tot
        b = int(round(acc * blocks))
        b = max(b, offs[-1] // ALIGN + 1)          # at least one block for rank q
        b = min(b, blocks - (R - 1 - q))            # and one for every later rank
        offs.append(b * ALIGN)
    offs.append(n)
    return offs


@dataclass
class AdamConfig:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0


@dataclass
class EngineConfig:
    compute_dtype: torch.dtype = torch.bfloat16
    reduce_dtype: torch.dtype = torch.float32
    optimizer_in_backward: bool = False
    offload_params: bool = False
    zero_level: int = 3
    collectives: str = "library"      # "library" (NCCL / gloo) | "fused" (in-kernel NVLink, CUDA only)
    grad_divide_by_group: bool = False  # reference arithmetic: mean over DP ranks
    adam: AdamConfig = field(default_factory=AdamConfig)
    seed: int = 0


class Streams:
    """Side streams shared by every unit of the process (several stages per rank share them,
    as in the reference, utils/patch.py:1017-1043)."""

    def __init__(self, device: torch.device):
        self.cuda = device.type == "cuda"
        if self.cuda:
            self.comm = torch.cuda.Stream(device=device)
            self.copy = torch.cuda.Stream(device=device)
        else:
            self.comm = self.copy = None
        self.measure_exposed = False
        self.exposed_events: list = []  # (start, end) pairs bracketing compute-stream waits on comm / p2p

    def wait_event(self, ev, kind: str = "zero") -> None:
        """Compute stream waits for `ev`; when measuring, the wait is bracketed by timing events so
        the time the compute stream sat idle on communication can be summed up after the step.
        `kind`: "zero" (gathers, reductions, optimizer, offload copies) or "pipeline" (a receive from
        the neighbouring stage: that wait also contains the time the neighbour needed to produce the
        tensor, i.e. the pipeline bubble, not only the transfer)."""
        cur = torch.cuda.current_stream()
        if not self.measure_exposed:
            cur.wait_event(ev)
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(cur)
        cur.wait_event(ev)
        b.record(cur)
        self.exposed_events.append((a, b, kind))

    def wait_stream(self, other, kind: str = "zero") -> None:
        cur = torch.cuda.current_stream()
        if not self.measure_exposed:
            cur.wait_stream(other)
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(cur)
        cur.wait_stream(other)
        b.record(cur)
        self.exposed_events.append((a, b, kind))

    def exposed_ms(self, clear: bool = True, by_kind: bool = False):
        """Sum of the bracketed waits (call after a device synchronisation); with `by_kind` a dict per kind."""
        out: dict = {}
        for a, b, kind in self.exposed_events:
            out[kind] = out.get(kind, 0.0) + a.elapsed_time(b)
        if clear:
            self.exposed_events.clear()
        return out if by_kind else sum(out.values())


@dataclass
class Counters:
    all_gathers: int = 0
    reduce_scatters: int = 0
    all_reduces: int = 0
    adam_steps: int = 0
    h2d_bytes: int = 0
    d2h_bytes: int = 0


class ZeroUnit:
    def __init__(self, layer: Layer, gid: int, *, device: torch.device, cfg: EngineConfig, ops, shard: Group,
                 replicate: Group, rank: int, streams: Streams, zero_level: Optional[int] = None,
                 counters: Optional[Counters] = None, meta_init: bool = False, shard_ratios=None,
                 tp_group: Optional[Group] = None):
        self.layer, self.gid, self.device, self.cfg, self.ops = layer, gid, device, cfg, ops
        # tensor-parallel lane of this rank: gradients of parameters every process of the lane holds
        # whole (norm weights, embedding, head, ...) are summed over it before the data-parallel reduction
        self.tp_group = tp_group if tp_group is not None and tp_group.size > 1 else None
        self.shard_group, self.rep_group, self.rank, self.streams = shard, replicate, rank, streams
        self.zero_level = zero_level or cfg.zero_level
        self.counters = counters or Counters()
        self.R = shard.size
        self.r = shard.index_of(rank)
        _, raw = layer.layout()
        q = self.R * ALIGN
        self.n = (raw + q - 1) // q * q
        self.offs = shard_bounds(self.n, self.R, shard_ratios if self.R > 1 else None)
        self.uneven = len({self.offs[q + 1] - self.offs[q] for q in range(self.R)}) > 1
        self.lo, self.hi = self.offs[self.r], self.offs[self.r + 1]
        self.shard_n = self.hi - self.lo
        self.cuda = device.type == "cuda"
        self.step_count = 0
        # ---- persistent state ------------------------------------------------------
        lo, hi = self.lo, self.hi
        full32 = torch.empty(self.n, dtype=torch.float32, device=device)
        if not meta_init:
            layer.init_flat(full32, cfg.seed * 1000003 + gid)
        self.master = full32[lo:hi].clone()
        del full32
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.p_shard = self.master.to(cfg.compute_dtype)
        self.grad_shard: Optional[torch.Tensor] = None  # reduced gradients awaiting optimizer_step
        # ---- transient state -------------------------------------------------------
        self.full: Optional[torch.Tensor] = None
        self.full_event = None
        self.grad: Optional[torch.Tensor] = None
        self.update_event = None
        # ---- offload ----------------------------------------------------------------
        self.host_master = self.host_p = None
        if cfg.offload_params:
            self._offload_init()
        if self.R == 1 and not cfg.offload_params:
            self.full = self.p_shard  # nothing to gather: the shard is the whole unit

    # ------------------------------------------------------------------ offload
    def _pinned(self, t: torch.Tensor) -> torch.Tensor:
        h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.cuda)
        h.copy_(t)
        return h

    def _offload_init(self):
        self.host_master = self._pinned(self.master)
        self.host_p = self._pinned(self.p_shard)
        self.master = None
        self.p_shard = None

    def _fetch_shard(self):
        """H2D of the bf16 shard on the copy stream; the comm stream waits for it."""
        if self.p_shard is not None or self.host_p is None:
            return
        if self.cuda:
            self.p_shard = torch.empty(self.shard_n, dtype=self.cfg.compute_dtype, device=self.device)
            self.streams.copy.wait_stream(torch.cuda.current_stream())
            with phase("offload.h2d_shard"), torch.cuda.stream(self.streams.copy):
                self.p_shard.copy_(self.host_p, non_blocking=True)
            self.p_shard.record_stream(self.streams.copy)
            self.streams.comm.wait_stream(self.streams.copy)
        else:
            self.p_shard = self.host_p.clone()
        self.counters.h2d_bytes += self.host_p.numel() * self.host_p.element_size()

    # ------------------------------------------------------------------ parameters
    def prefetch(self):
        """Issues the all-gather (no-op if the unsharded buffer exists or is in flight)."""
        if self.full is not None:
            return
        self._fetch_shard()
        if self.R == 1:
            if self.cuda and self.host_p is not None:
                ev = torch.cuda.Event()
                ev.record(self.streams.copy)
                self.full_event = ev
            self.full = self.p_shard
            return
        full = torch.empty(self.n, dtype=self.cfg.compute_dtype, device=self.device)
        self.counters.all_gathers += 1
        if self.cuda:
            cur = torch.cuda.current_stream()
            self.streams.comm.wait_stream(cur)
            with phase("zero.all_gather"), torch.cuda.stream(self.streams.comm):
                if self.update_event is not None:
                    self.streams.comm.wait_event(self.update_event)
                SC.read(("shard", id(self)), label="all-gather of the bf16 shard")
                self._gather_into(full, self.p_shard)
                SC.wrote(("full", id(self)))
                ev = torch.cuda.Event()
                ev.record(self.streams.comm)
            full.record_stream(self.streams.comm)
            self.full_event = ev
        else:
            self._gather_into(full, self.p_shard)
        self.full = full
        if self.host_p is not None:
            self.p_shard = None  # the device copy of an offloaded shard lives only for the gather

    def _gather_into(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        pg = self.shard_group.pg
        if not self.uneven:
            dist.all_gather_into_tensor(full, shard, group=pg)
            return
        full[self.lo:self.hi].copy_(shard)
        for q, owner in enumerate(self.shard_group.ranks):
            dist.broadcast(full[self.offs[q]:self.offs[q + 1]], src=owner, group=pg)

    def _reduce_scatter(self, g_full: torch.Tensor) -> torch.Tensor:
        pg = self.shard_group.pg
        if not self.uneven:
            g_sh = torch.empty(self.shard_n, dtype=g_full.dtype, device=self.device)
            dist.reduce_scatter_tensor(g_sh, g_full, group=pg)
            return g_sh
        for q, owner in enumerate(self.shard_group.ranks):
            dist.reduce(g_full[self.offs[q]:self.offs[q + 1]], dst=owner, group=pg)
        return g_full[self.lo:self.hi]

    def acquire(self) -> None:
        """Makes the unsharded parameters available to the compute stream and binds the layer."""
        self.prefetch()
        if self.cuda and self.full_event is not None:
            with phase("zero.wait_params"):
                self.streams.wait_event(self.full_event)
            self.full_event = None
        if self.cuda:
            SC.read(("full", id(self)), label="layer compute on gathered parameters")
        self.layer.bind(self.full, self.grad)

    def release(self, force: bool = False) -> None:
        """Frees the unsharded buffer (ZeRO-3, or any level with force=True)."""
        if self.full is None:
            return
        if self.R == 1 and self.host_p is None:
            return
        if self.zero_level == 2 and not force:
            return
        if self.R == 1:
            self.p_shard = None
        self.full = None
        self.layer.bind(None, self.grad)

    # ------------------------------------------------------------------ gradients
    def grad_views(self) -> None:
        if self.grad is None:
            self.grad = torch.zeros(self.n, dtype=self.cfg.reduce_dtype, device=self.device)
        if self.cuda:
            SC.wrote(("grad", id(self)))   # backward kernels on the current stream accumulate into it
        self.layer.bind(self.full, self.grad)

    def _adam(self, g: torch.Tensor, grad_scale: float):
        cfg = self.cfg.adam
        self.step_count += 1
        offl = self.host_master is not None
        if offl:
            master = self.host_master.to(self.device, non_blocking=True)
            p16 = torch.empty(self.shard_n, dtype=self.cfg.compute_dtype, device=self.device)
            self.counters.h2d_bytes += self.host_master.numel() * 4
        else:
            master, p16 = self.master, self.p_shard
        self.ops.adam_step(master, self.m, self.v, g, p16, lr=cfg.lr, beta1=cfg.beta1, beta2=cfg.beta2, eps=cfg.eps,
                           weight_decay=cfg.weight_decay, step=self.step_count, grad_scale=grad_scale)
        self.counters.adam_steps += 1
        if offl:
            self.host_master.copy_(master, non_blocking=True)
            self.host_p.copy_(p16, non_blocking=True)
            self.counters.d2h_bytes += self.host_master.numel() * 4 + self.host_p.numel() * self.host_p.element_size()

    def reduce_grads(self) -> None:
        """Call once per step after the unit's last backward microbatch."""
        if self.grad is None:
            return
        g_full = self.grad
        self.grad = None
        self.layer.bind(self.full, None)
        gscale = 1.0 / self.R if self.cfg.grad_divide_by_group else 1.0
        if self.rep_group.size > 1 and self.cfg.grad_divide_by_group:
            gscale /= self.rep_group.size

        def work():
            if self.tp_group is not None:
                from ..models.tp_layers import replicated_ranges

                for o, k in replicated_ranges(self.layer):
                    dist.all_reduce(g_full[o:o + k], group=self.tp_group.pg)
                    self.counters.all_reduces += 1
            if self.R > 1:
                g_sh = self._reduce_scatter(g_full)
                self.counters.reduce_scatters += 1
            else:
                g_sh = g_full
            if self.rep_group.size > 1:
                dist.all_reduce(g_sh, group=self.rep_group.pg)
                self.counters.all_reduces += 1
            if self.cfg.optimizer_in_backward:
                self._adam(g_sh, gscale)
            else:
                self.grad_shard = g_sh  # consumed (with its scale) by optimizer_step
                self.grad_shard_scale = gscale
            return g_sh

        if self.cuda:
            cur = torch.cuda.current_stream()
            self.streams.comm.wait_stream(cur)
            with phase("zero.reduce_scatter"), torch.cuda.stream(self.streams.comm):
                SC.read(("grad", id(self)), label="reduce-scatter of the gradient bucket")
                g_sh = work()
                if self.cfg.optimizer_in_backward:
                    SC.wrote(("shard", id(self)))
                ev = torch.cuda.Event()
                ev.record(self.streams.comm)
            g_full.record_stream(self.streams.comm)
            g_sh.record_stream(self.streams.comm)
            self.update_event = ev
        else:
            work()
        if self.cfg.optimizer_in_backward:
            self._after_update()

    def _after_update(self):
        """The bf16 shard changed: any unsharded copy is stale."""
        if self.R == 1 and self.host_p is None:
            self.full = self.p_shard
        else:
            self.full = None
            self.full_event = None
            if self.host_p is not None:
                self.p_shard = None

    def optimizer_step(self) -> None:
        """Adam on the accumulated gradient shard (used when not optimizer-in-backward)."""
        if self.grad_shard is None:
            return
        g = self.grad_shard
        self.grad_shard = None
        if self.cuda:
            cur = torch.cuda.current_stream()
            if self.update_event is not None:
                cur.wait_event(self.update_event)
            with phase("zero.adam"):
                self._adam(g, getattr(self, 'grad_shard_scale', 1.0))
            SC.wrote(("shard", id(self)))
            ev = torch.cuda.Event()
            ev.record(cur)
            self.update_event = ev
        else:
            self._adam(g, getattr(self, 'grad_shard_scale', 1.0))
        self._after_update()

    def finish_step(self) -> None:
        """End of step: ZeRO-2 units drop their now stale unsharded parameters."""
        if self.R > 1 or self.host_p is not None:
            self.full = None
            self.full_event = None

    # ------------------------------------------------------------------ introspection
    def full_master(self) -> torch.Tensor:
        """fp32 master parameters of the whole unit gathered on every rank (tests, checkpoints)."""
        mine = self.master if self.master is not None else self.host_master.to(self.device)
        if self.cuda:
            torch.cuda.synchronize()
        if self.R == 1:
            return mine.clone()
        out = torch.empty(self.n, dtype=torch.float32, device=self.device)
        self._gather_into(out, mine.contiguous())
        return out

    def state_tensors(self) -> dict[str, torch.Tensor]:
        mine = self.master if self.master is not None else self.host_master
        return {"master": mine, "m": self.m, "v": self.v}

    def load_state(self, master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int) -> None:
        if self.host_master is not None:
            self.host_master.copy_(master)
            self.host_p.copy_(master.to(self.cfg.compute_dtype))
        else:
            self.master.copy_(master)
            self.p_shard.copy_(self.master.to(self.cfg.compute_dtype))
        self.m.copy_(m)
        self.v.copy_(v)
        self.step_count = step
        self._after_update()


class StageEngine:
    """All ZeRO units of one pipeline stage on this rank, in layer order."""

    def __init__(self, layers: list[Layer], gids: list[int], *, device, cfg: EngineConfig, ops, shard: Group,
                 replicate: Group, rank: int, streams: Optional[Streams] = None, zero_level: Optional[int] = None,
                 meta_init: bool = False, shard_ratios=None, tp_group: Optional[Group] = None):
        self.device, self.cfg, self.ops = device, cfg, ops
        self.streams = streams or Streams(device)
        self.counters = Counters()
        cls = ZeroUnit
        kw = {}
        if tp_group is not None and tp_group.size > 1:
            kw["tp_group"] = tp_group     # the fused unit does not cover tensor-parallel lanes
        elif (cfg.collectives == "fused" and device.type == "cuda" and shard.size > 1 and replicate.size == 1
                and shard_ratios is None):
            from .fused import FusedZeroUnit

            cls = FusedZeroUnit
        self.units = [cls(ly, gid, device=device, cfg=cfg, ops=ops, shard=shard, replicate=replicate, rank=rank,
                          streams=self.streams, zero_level=zero_level, counters=self.counters, meta_init=meta_init,
                          shard_ratios=shard_ratios, **kw)
                      for ly, gid in zip(layers, gids)]

    def __len__(self):
        return len(self.units)

    def __getitem__(self, i) -> ZeroUnit:
        return self.units[i]

    def prefetch_all(self, reverse: bool = False) -> None:
        for u in (reversed(self.units) if reverse else self.units):
            u.prefetch()

    def optimizer_step(self) -> None:
        for u in self.units:
            u.optimizer_step()

    def finish_step(self) -> None:
        for u in self.units:
            u.finish_step()
        if self.device.type == "cuda":
            self.streams.wait_stream(self.streams.comm)

    def num_params(self) -> int:
        return sum(u.layer.num_params() for u in self.units)
