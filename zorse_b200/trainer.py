"""Builds the whole training job of one rank from a `PipelineConfig` and runs steps.

This is the public API behind `zorse.py` (and what `bench.py` times end to end):

    trainer = Trainer(cfg, TrainerOptions(...))       # groups, plan, stages, engine, schedule
    batch = trainer.synthetic_batch()                 # pinned host token ids / labels
    loss = trainer.train_step_from_host(batch)        # H2D copy, schedule.step, loss read-back

Call stack parity with the reference trainer (zorse.py:212-283): dist init -> parse config ->
build stages (+ communicators, static plan) -> wrap each stage in the ZeRO engine -> pick a
schedule -> loop over `schedule.step`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist

from .config.training_config import PipelineConfig, dtype_from_str
from .engine.zero import AdamConfig, EngineConfig, Streams
from .models import registry
from .ops.api import default_ops_for, get_ops
from .parallel import groups as G
from .parallel.p2p import GlooP2P, LaneTransport, LocalMailbox, make_transport
from .parallel.p2p_plan import create_static_comm_plans, is_regular
from .parallel.schedules import build_schedule
from .parallel.stage import PipelineStage
from .utils import canary


@dataclass
class TrainerOptions:
    schedule: str = "layer_major"
    ops: Optional[str] = None              # "sm100" | "ref"; default by device
    optimizer_in_backward: bool = False
    offload_model_params: bool = False
    gloo_p2p: bool = False
    collectives: str = "library"           # "library" | "fused"
    activation_recompute: Optional[bool] = None
    activation_offload: Optional[bool] = None
    lr: float = 1e-3
    seed: int = 0
    backend: Optional[str] = None          # torch.distributed backend override ("gloo" forces CPU)
    model_overrides: dict = field(default_factory=dict)
    pipeline_log: object = None
    defer_wgrad: bool = False              # 1F1B: input gradients are sent upstream before the weight-gradient GEMMs run
    defer_tail_wgrad: int = 0              # 1F1B, last stage: head (+ this many - 1 blocks) weight gradients after its last backward; 0 = off
    p2p_timeout_s: Optional[float] = None  # Gloo p2p: a receive that waits longer raises, naming the missing message
    p2p_fault_hooks: bool = False          # wrap the transport so that tests can drop or delay messages (host side)
    prepost_recv: bool = False             # 1F1B: post the next operation's receive ahead (per-boundary p2p groups)
    shift_labels: bool = False             # synthetic targets = next token of the inputs (last position ignored)


class Trainer:
    def __init__(self, cfg: PipelineConfig, opt: TrainerOptions):
        if opt.offload_model_params and not opt.optimizer_in_backward:
            raise ValueError("--offload_model_params requires --optimizer_in_backwards")
        if opt.collectives == "fused":
            opt.optimizer_in_backward = True  # the fused reduce-scatter kernel applies Adam itself
        self.cfg, self.opt = cfg, opt
        self.device = G.dist_init(opt.backend)
        self.rank, self.world = G.rank(), G.world_size()
        need = cfg.world_size
        if need != self.world:
            raise ValueError(f"the training config names {need} ranks but the job has {self.world}")
        self.ops = get_ops(opt.ops or default_ops_for(self.device))
        compute = dtype_from_str(cfg.autocast_dtype)
        if self.ops.name == "sm100" and compute != torch.bfloat16:
            raise ValueError("the sm100 kernels compute in bfloat16; set autocast_dtype to bfloat16")
        self.engine_cfg = EngineConfig(
            compute_dtype=compute, reduce_dtype=dtype_from_str(cfg.reduce_dtype),
            optimizer_in_backward=opt.optimizer_in_backward, offload_params=opt.offload_model_params,
            collectives=opt.collectives, grad_divide_by_group=cfg.grad_norm_compat == "reference",
            adam=AdamConfig(lr=opt.lr), seed=opt.seed)
        self.streams = Streams(self.device)
        # tensor parallelism: the config numbers lanes of tp processes; everything that follows the plan
        # (stages, microbatches, p2p peers) uses the lane number, the groups use process ranks
        tp = cfg.tensor_parallel_size
        if tp > 1 and opt.collectives == "fused":
            import warnings

            warnings.warn("fused ZeRO collectives do not cover tensor-parallel lanes: their units use the library "
                          "collectives (the lane's own fused kernels are selected with ZORSE_TP_FUSED=1)")
        self.lane, self.tp_index = self.rank // tp, self.rank % tp
        stage_groups = G.StageGroups.create_all(cfg.stages, self.rank, tp=tp)
        self.gloo_group = G.gloo_world_group() if (opt.gloo_p2p or self.device.type == "cuda") and G.is_dist() else None
        # --gloo_p2p on GPUs: keep an NCCL transport next to the Gloo one so that the ZeRO-2 schedule
        # can alternate between them by stage width; on CPU ranks there is only Gloo
        both = opt.gloo_p2p and self.device.type == "cuda" and G.is_dist()
        self.transport = make_transport(self.device, use_gloo=opt.gloo_p2p and not both, gloo_group=self.gloo_group,
                                        streams=self.streams, split_parity=not is_regular(cfg) or opt.prepost_recv,
                                        recv_timeout_s=opt.p2p_timeout_s)
        if opt.p2p_fault_hooks:
            from .parallel.p2p import FaultyTransport

            self.transport = self.fault_transport = FaultyTransport(self.transport)
        self.gloo_transport = GlooP2P(self.device, self.gloo_group, recv_timeout_s=opt.p2p_timeout_s) if both else None
        if tp > 1:
            self.transport = LaneTransport(self.transport, tp, self.tp_index)
            if self.gloo_transport is not None:
                self.gloo_transport = LaneTransport(self.gloo_transport, tp, self.tp_index)
        if cfg.comm_plan == "latency" and not cfg.rank_latency_ms:
            cfg.rank_latency_ms = self._rank_latencies(cfg, tp)
        plans = create_static_comm_plans(cfg)
        self.plan = plans.get(self.lane)     # None on a rank the plan leaves idle
        offload_act = cfg.activation_offload if opt.activation_offload is None else opt.activation_offload
        mailbox = LocalMailbox()     # hand-offs between two stages of this rank never touch a transport
        self.stages = [
            PipelineStage(cfg, st, rank=self.lane, process_rank=self.rank, device=self.device, ops=self.ops,
                          engine_cfg=self.engine_cfg,
                          groups=stage_groups[st.stage_id], streams=self.streams, pattern=self.plan.stages[st.stage_id],
                          transport=self.transport, gloo_transport=self.gloo_transport,
                          activation_offload=bool(offload_act),
                          model_overrides=opt.model_overrides, local_mailbox=mailbox,
                          split_parity=True if opt.prepost_recv else None)
            for st in cfg.stages_of_rank(self.lane)]
        self.spec = (self.stages[0].spec if self.stages else
                     registry.get_spec(cfg.model_name, vocab=cfg.vocab_size, **(opt.model_overrides or {})))
        recompute = cfg.activation_recompute if opt.activation_recompute is None else opt.activation_recompute
        name = cfg.schedule or opt.schedule
        self.schedule = build_schedule(name, self.stages, cfg, recompute=recompute, pipeline_log=opt.pipeline_log,
                                       defer_wgrad=opt.defer_wgrad,
                                       defer_tail_wgrad=opt.defer_tail_wgrad or cfg.defer_tail_wgrad or 0,
                                       prepost_recv=opt.prepost_recv)
        self.step_idx = 0

    # ------------------------------------------------------------------ data
    def synthetic_batch(self, seed: Optional[int] = None, pin: bool = True) -> dict:
        """Uniform random token ids and labels for the whole global batch, [M, B, S] int64 on
        the host (pinned when a GPU is used) — the reference trains on exactly this kind of data,
        generated once and reused every step (zorse.py:42-47, 73-85)."""
        cfg = self.cfg
        g = torch.Generator().manual_seed(cfg_seed(self.opt.seed if seed is None else seed))
        M, B, S = cfg.num_microbatches, cfg.microbatch_size, cfg.sequence_length
        spec = self.spec
        if spec.family == "vit":
            x = torch.randn(M, B, 3, spec.image, spec.image, generator=g)
            y = torch.randint(0, spec.classes, (M, B), generator=g)
        else:
            x = torch.randint(0, cfg.vocab_size, (M, B, S), generator=g)
            y = torch.randint(0, cfg.vocab_size, (M, B, S), generator=g)
            if self.opt.shift_labels:
                from .utils.data import shift_labels

                y = shift_labels(x)
        if pin and self.device.type == "cuda":
            x, y = x.pin_memory(), y.pin_memory()
        return {"inputs": x, "targets": y}

    def needed_microbatches(self):
        first = sorted({g for st in self.stages if st.is_first for g in st.microbatches})
        last = sorted({g for st in self.stages if st.is_last for g in st.microbatches})
        return first, last

    def to_device(self, batch: dict):
        """Copies the microbatches this rank consumes to its device. Returns (inputs, targets,
        bytes copied)."""
        first, last = self.needed_microbatches()
        inputs, targets, nbytes = {}, {}, 0
        for g in first:
            t = batch["inputs"][g]
            inputs[g] = t.to(self.device, non_blocking=True)
            nbytes += t.numel() * t.element_size()
        for g in last:
            t = batch["targets"][g]
            targets[g] = t.to(self.device, non_blocking=True)
            nbytes += t.numel() * t.element_size()
        return inputs, targets, nbytes

    # ------------------------------------------------------------------ steps
    def train_step(self, inputs: dict, targets: dict):
        """One optimizer step on device-resident microbatches. Returns this rank's share of
        the mean loss as a device scalar (None on ranks without the last stage)."""
        loss = self.schedule.step(self.step_idx, inputs, targets)
        self.step_idx += 1
        if canary.enabled():
            self.synchronize()
            canary.check_all()     # raises if a guard band next to a raw-pointer buffer changed
        return loss

    def train_step_from_host(self, batch: dict) -> Optional[float]:
        """Host-to-device copy of this step's inputs, one step, device-to-host read of the loss."""
        inputs, targets, _ = self.to_device(batch)
        loss = self.train_step(inputs, targets)
        return None if loss is None else float(loss.item())

    def global_loss(self, loss) -> float:
        """Sum of the last-stage ranks' loss shares (= mean loss of the global batch)."""
        v = torch.zeros(1, dtype=torch.float64)
        if loss is not None:
            v[0] = float(loss)
        if not G.is_dist():
            return float(v[0])
        if self.gloo_group is not None:
            dist.all_reduce(v, group=self.gloo_group)
        elif dist.get_backend() == "gloo":
            dist.all_reduce(v)
        else:
            t = v.to(self.device)
            dist.all_reduce(t)
            v = t.cpu()
        return float(v[0])

    def _rank_latencies(self, cfg, tp: int) -> dict:
        """ms per layer and microbatch of every rank of the plan, for the latency-driven microbatch routing: every
        process reports its GPU model, the profile table (data/model_latencies.json) gives forward + backward time of
        one block of this model on that GPU (reference zorse_utils/pipeline_comm.py:176-191, 214-226)."""
        from .planner.latency import load_model_compute_latencies_per_gpu
        from .utils.metrics import clean_gpu_name

        name = clean_gpu_name(torch.cuda.get_device_name(self.device)) if self.device.type == "cuda" else "cpu"
        names = [name] * self.world
        if G.is_dist():
            names = [None] * self.world
            dist.all_gather_object(names, name, group=self.gloo_group)
        lat = load_model_compute_latencies_per_gpu(cfg.model_name, sorted(set(names)), cfg.sequence_length,
                                                   cfg.autocast_dtype, cfg.microbatch_size)
        return {lane: lat[names[lane * tp]].total for lane in range(self.world // tp)}

    def measure_exposed_comm(self, on: bool = True) -> None:
        """Brackets every compute-stream wait on a collective or a p2p receive with timing events."""
        self.streams.measure_exposed = on and self.device.type == "cuda"
        self.streams.exposed_events.clear()

    def exposed_comm_ms(self) -> float:
        """Time the compute stream spent blocked on communication since the last call (ms)."""
        self.synchronize()
        return self.streams.exposed_ms() if self.device.type == "cuda" else 0.0

    def exposed_comm_breakdown(self) -> dict:
        """The same time split by cause (ms): `zero` = waits on gathers, reductions, optimizer and offload
        copies; `pipeline` = waits on receives from the neighbouring stage, which contain the time that
        stage needed to produce the tensor (the pipeline bubble) as well as the transfer."""
        self.synchronize()
        d = self.streams.exposed_ms(by_kind=True) if self.device.type == "cuda" else {}
        return {"zero": float(d.get("zero", 0.0)), "pipeline": float(d.get("pipeline", 0.0))}

    def synchronize(self):
        if self.device.type == "cuda":
            torch.cuda.synchronize()

    def barrier(self):
        if G.is_dist():
            if self.gloo_group is not None:
                dist.barrier(group=self.gloo_group)
            else:
                dist.barrier()

    def check_kernels(self):
        if self.ops.name == "sm100":
            self.ops.k.check_status(self.device)

    def num_params(self) -> int:
        return sum(st.engine.num_params() for st in self.stages)

    def counters(self):
        return [st.engine.counters for st in self.stages]


def cfg_seed(seed: int) -> int:
    return 7919 * (seed + 1)
