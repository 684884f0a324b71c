"""Typed view of `training_config.json` (planner output = trainer input).

Same keys, defaults and validation rules as the reference reader
(zorse_utils/pipeline_config.py:8-207): stages may be listed in any order and are
sorted by the start of their layer range, the ranges must tile `[0, L)` without gaps,
`global_batch_size = microbatch_size * sum(num_microbatches_per_rank)` for every
stage, and `zero_config` lists the shard groups of a stage (more than one group =
hybrid shard: reduce-scatter inside a group, all-reduce across groups).

Additions over the reference format (all optional, defaults keep reference behaviour):
`zero_level` per stage (2 or 3), `shard_ratio` per stage (relative parameter-shard sizes of
the ranks of a shard group, e.g. by GPU memory; the reference's dormant `split_uneven` /
`shard_ratio` state, utils/patch.py:308-441), `reduce_dtype`, `schedule`,
`activation_recompute`, `activation_offload`, `grad_norm_compat`, and `tensor_parallel_size`
(tp, default 1).  With tp > 1 every rank number in the file names a *lane* of tp consecutive
processes (lane l = ranks l*tp .. l*tp + tp - 1, which hold the tensor-parallel slices of the
lane's layers); the job then has tp times as many processes as the file names lanes.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional, Sequence

DTYPE_NAMES = ("float16", "bfloat16", "float32")


class ConfigError(ValueError):
    pass


def dtype_from_str(name: str):
    import torch

    table = {"float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
             "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
             "float32": torch.float32, "fp32": torch.float32, "float": torch.float32}
    if name not in table:
        raise ConfigError(f"unknown dtype {name!r}; expected one of {sorted(table)}")
    return table[name]


def dtype_to_str(dtype) -> str:
    return str(dtype).replace("torch.", "")


@dataclass
class StageConfig:
    stage_id: int
    gpu_ranks: tuple[int, ...]
    layer_partition: tuple[int, int]
    microbatch_size: int
    zero_config: tuple[tuple[int, ...], ...]
    num_microbatches_per_rank: tuple[int, ...]
    zero_level: int = 3
    shard_ratio: Optional[tuple[float, ...]] = None   # one entry per rank of a shard group

    @property
    def num_microbatches(self) -> int:
        return sum(self.num_microbatches_per_rank)

    @property
    def num_layers(self) -> int:
        return self.layer_partition[1] - self.layer_partition[0]

    def shard_group_of(self, rank: int) -> tuple[int, ...]:
        for g in self.zero_config:
            if rank in g:
                return g
        raise ConfigError(f"rank {rank} not in zero_config of stage {self.stage_id}")

    def replicate_group_of(self, rank: int) -> tuple[int, ...]:
        """The j-th members of every shard group, j = position of `rank` in its group."""
        g = self.shard_group_of(rank)
        j = g.index(rank)
        return tuple(grp[j] for grp in self.zero_config)

    def validate(self) -> None:
        s = f"stage {self.stage_id}"
        if not self.gpu_ranks:
            raise ConfigError(f"{s}: gpu_ranks is empty")
        if len(set(self.gpu_ranks)) != len(self.gpu_ranks):
            raise ConfigError(f"{s}: duplicate ranks in gpu_ranks {self.gpu_ranks}")
        if len(self.num_microbatches_per_rank) != len(self.gpu_ranks):
            raise ConfigError(f"{s}: num_microbatches_per_rank has {len(self.num_microbatches_per_rank)} "
                              f"entries for {len(self.gpu_ranks)} ranks")
        if any(m < 0 for m in self.num_microbatches_per_rank):
            raise ConfigError(f"{s}: negative microbatch count")
        a, b = self.layer_partition
        if a < 0 or b <= a:
            raise ConfigError(f"{s}: bad layer_partition {self.layer_partition}")
        if self.microbatch_size <= 0:
            raise ConfigError(f"{s}: microbatch_size must be positive")
        flat = [r for g in self.zero_config for r in g]
        if sorted(flat) != sorted(self.gpu_ranks):
            raise ConfigError(f"{s}: zero_config {self.zero_config} does not partition gpu_ranks {self.gpu_ranks}")
        sizes = {len(g) for g in self.zero_config}
        if len(sizes) != 1:
            raise ConfigError(f"{s}: shard groups of different sizes {self.zero_config}")
        if self.zero_level not in (2, 3):
            raise ConfigError(f"{s}: zero_level must be 2 or 3")
        if self.shard_ratio is not None:
            if len(self.shard_ratio) != len(self.zero_config[0]) or any(x <= 0 for x in self.shard_ratio):
                raise ConfigError(f"{s}: shard_ratio needs one positive entry per rank of a shard group")


@dataclass
class PipelineConfig:
    model_name: str
    global_batch_size: int
    microbatch_size: int
    sequence_length: int
    stages: list[StageConfig]
    vocab_size: int = 49152
    fused_optimizer: bool = True
    interleave_degree: int = 1
    latency: Optional[float] = None
    autocast_dtype: str = "bfloat16"
    reduce_dtype: str = "float32"
    split_microbatches_evenly: bool = False
    sync_after_recompute: bool = False
    interleave_stage_sync: bool = False
    gloo_batch_recv: bool = True
    alternate_nccl_gloo: bool = True
    # accepted for compatibility: the reference builds non-leader ranks' models on the meta device when set
    # (zorse_utils/pipeline.py:205-226); here every unit is always initialised on its own, on the device,
    # and only the rank's shard is kept, so no rank ever holds more than one whole layer in fp32
    large_model_init: bool = False
    # extensions
    schedule: Optional[str] = None
    activation_recompute: Optional[bool] = None
    activation_offload: Optional[bool] = None
    grad_norm_compat: str = "mean"
    unused_ranks: tuple[int, ...] = ()   # ranks of the job that own no stage (the planner may leave a slow GPU out)
    tensor_parallel_size: int = 1        # processes per rank number of this file (see the module docstring)
    # "interleave": microbatches are dealt to a stage's ranks by their counts alone; "latency": by the ranks'
    # per-layer latencies as well (reference zorse_utils/pipeline_comm.py:193-303), from `rank_latency_ms`
    # (rank -> ms per layer and microbatch) or, when absent, from the profile table and the ranks' GPU models
    comm_plan: str = "interleave"
    rank_latency_ms: Optional[dict] = None
    # 1F1B: weight gradients of the last stage's last N layers (the head first) run after its last backward
    # (schedules/one_f_one_b.py); written by the planner when asked for a 1F1B plan, a trainer flag overrides it
    defer_tail_wgrad: Optional[int] = None
    extra: dict = field(default_factory=dict)

    @property
    def num_microbatches(self) -> int:
        return self.global_batch_size // self.microbatch_size

    @property
    def num_layers(self) -> int:
        return max(s.layer_partition[1] for s in self.stages)

    @property
    def num_lanes(self) -> int:
        return len({r for s in self.stages for r in s.gpu_ranks} | set(self.unused_ranks))

    @property
    def world_size(self) -> int:
        return self.num_lanes * self.tensor_parallel_size

    @property
    def gpu_groups(self) -> list[tuple[int, ...]]:
        seen: list[tuple[int, ...]] = []
        for s in self.stages:
            if s.gpu_ranks not in seen:
                seen.append(s.gpu_ranks)
        return seen

    def stages_of_rank(self, rank: int) -> list[StageConfig]:
        return [s for s in self.stages if rank in s.gpu_ranks]

    def validate(self) -> None:
        if self.global_batch_size <= 0 or self.microbatch_size <= 0 or self.sequence_length <= 0:
            raise ConfigError("global_batch_size, microbatch_size and sequence_length must be positive")
        if self.global_batch_size % self.microbatch_size:
            raise ConfigError(f"global_batch_size {self.global_batch_size} is not a multiple of "
                              f"microbatch_size {self.microbatch_size}")
        if self.autocast_dtype not in DTYPE_NAMES or self.reduce_dtype not in DTYPE_NAMES:
            raise ConfigError("autocast_dtype / reduce_dtype must be one of " + ", ".join(DTYPE_NAMES))
        if not self.stages:
            raise ConfigError("pipeline_config is empty")
        if self.tensor_parallel_size < 1:
            raise ConfigError("tensor_parallel_size must be at least 1")
        for s in self.stages:
            s.validate()
            if s.num_microbatches != self.num_microbatches:
                raise ConfigError(f"stage {s.stage_id}: {s.num_microbatches} microbatches, expected "
                                  f"{self.num_microbatches} (= global_batch_size / microbatch_size)")
        check_contiguous([s.layer_partition for s in self.stages])
        named = {r for s in self.stages for r in s.gpu_ranks}
        if named & set(self.unused_ranks):
            raise ConfigError(f"unused_ranks {sorted(named & set(self.unused_ranks))} also own stages")
        if sorted(named | set(self.unused_ranks)) != list(range(len(named) + len(self.unused_ranks))):
            raise ConfigError("the ranks named by the stages and by unused_ranks must be 0 .. world_size - 1")


def check_contiguous(parts: Sequence[tuple[int, int]]) -> None:
    """Layer ranges, sorted by start, must begin at 0 and follow one another without gap or overlap."""
    parts = sorted(parts)
    if parts[0][0] != 0:
        raise ConfigError(f"first layer range starts at {parts[0][0]}, expected 0")
    for (a0, a1), (b0, b1) in zip(parts, parts[1:]):
        if b0 != a1:
            raise ConfigError(f"layer ranges not contiguous: [{a0},{a1}) then [{b0},{b1})")


def split_evenly(total: int, n: int) -> tuple[int, ...]:
    base, rem = divmod(total, n)
    return tuple(base + (1 if i < rem else 0) for i in range(n))


def parse_pipeline_dict(d: dict[str, Any]) -> PipelineConfig:
    required = ("model_name", "global_batch_size", "microbatch_size", "sequence_length", "pipeline_config")
    for k in required:
        if k not in d:
            raise ConfigError(f"training config lacks required key {k!r}")
    gbs, mbs = int(d["global_batch_size"]), int(d["microbatch_size"])
    even = bool(d.get("split_microbatches_evenly", False))
    raw = sorted(d["pipeline_config"], key=lambda s: s["layer_partition"][0])
    stages = []
    for i, s in enumerate(raw):
        ranks = tuple(int(r) for r in s["gpu_ranks"])
        zc = s.get("zero_config") or [list(ranks)]
        if even or "num_microbatches_per_rank" not in s:
            per_rank = split_evenly(gbs // mbs, len(ranks))
        else:
            per_rank = tuple(int(m) for m in s["num_microbatches_per_rank"])
        stages.append(StageConfig(
            stage_id=i, gpu_ranks=ranks, layer_partition=(int(s["layer_partition"][0]), int(s["layer_partition"][1])),
            microbatch_size=mbs, zero_config=tuple(tuple(int(r) for r in g) for g in zc),
            num_microbatches_per_rank=per_rank, zero_level=int(s.get("zero_level", d.get("zero_level", 3))),
            shard_ratio=tuple(float(x) for x in s["shard_ratio"]) if s.get("shard_ratio") else None))
    known = {"model_name", "global_batch_size", "microbatch_size", "sequence_length", "pipeline_config", "vocab_size",
             "fused_optimizer", "interleave_degree", "latency", "autocast_dtype", "reduce_dtype",
             "split_microbatches_evenly", "skip_compute_sync", "interleave_stage_sync", "gloo_batch_recv",
             "alternate_nccl_gloo", "large_model_init", "schedule", "activation_recompute", "activation_offload",
             "grad_norm_compat", "zero_level", "unused_ranks", "tensor_parallel_size", "comm_plan", "rank_latency_ms",
             "defer_tail_wgrad"}
    cfg = PipelineConfig(
        model_name=str(d["model_name"]), global_batch_size=gbs, microbatch_size=mbs,
        sequence_length=int(d["sequence_length"]), stages=stages, vocab_size=int(d.get("vocab_size", 49152)),
        fused_optimizer=bool(d.get("fused_optimizer", True)), interleave_degree=int(d.get("interleave_degree", 1)),
        latency=d.get("latency"), autocast_dtype=str(d.get("autocast_dtype", "bfloat16")),
        reduce_dtype=str(d.get("reduce_dtype", "float32")), split_microbatches_evenly=even,
        sync_after_recompute=not bool(d.get("skip_compute_sync", True)),
        interleave_stage_sync=bool(d.get("interleave_stage_sync", False)),
        gloo_batch_recv=bool(d.get("gloo_batch_recv", True)), alternate_nccl_gloo=bool(d.get("alternate_nccl_gloo", True)),
        large_model_init=bool(d.get("large_model_init", False)), schedule=d.get("schedule"),
        activation_recompute=d.get("activation_recompute"), activation_offload=d.get("activation_offload"),
        grad_norm_compat=str(d.get("grad_norm_compat", "mean")),
        unused_ranks=tuple(int(r) for r in d.get("unused_ranks", ())),
        tensor_parallel_size=int(d.get("tensor_parallel_size", 1)),
        comm_plan=str(d.get("comm_plan", "interleave")),
        rank_latency_ms={int(k): float(v) for k, v in d["rank_latency_ms"].items()} if d.get("rank_latency_ms") else None,
        defer_tail_wgrad=int(d["defer_tail_wgrad"]) if d.get("defer_tail_wgrad") is not None else None,
        extra={k: v for k, v in d.items() if k not in known})
    cfg.validate()
    return cfg


def parse_pipeline_config(path: str | Path) -> PipelineConfig:
    with open(path) as f:
        return parse_pipeline_dict(json.load(f))


def to_dict(cfg: PipelineConfig) -> dict[str, Any]:
    """Inverse of parse_pipeline_dict: the JSON layout the planner writes."""
    d: dict[str, Any] = {
        "model_name": cfg.model_name, "global_batch_size": cfg.global_batch_size,
        "microbatch_size": cfg.microbatch_size, "sequence_length": cfg.sequence_length,
        "vocab_size": cfg.vocab_size, "fused_optimizer": cfg.fused_optimizer,
        "interleave_degree": cfg.interleave_degree, "latency": cfg.latency,
        "autocast_dtype": cfg.autocast_dtype, "reduce_dtype": cfg.reduce_dtype,
        "pipeline_config": [
            {"gpu_ranks": list(s.gpu_ranks), "num_microbatches_per_rank": list(s.num_microbatches_per_rank),
             "layer_partition": list(s.layer_partition), "zero_config": [list(g) for g in s.zero_config],
             **({"zero_level": s.zero_level} if s.zero_level != 3 else {}),
             **({"shard_ratio": list(s.shard_ratio)} if s.shard_ratio else {})}
            for s in cfg.stages],
    }
    if cfg.unused_ranks:
        d["unused_ranks"] = list(cfg.unused_ranks)
    if cfg.tensor_parallel_size != 1:
        d["tensor_parallel_size"] = cfg.tensor_parallel_size
    if cfg.split_microbatches_evenly:
        d["split_microbatches_evenly"] = True
    if cfg.sync_after_recompute:
        d["skip_compute_sync"] = False
    for k in ("interleave_stage_sync", "large_model_init"):
        if getattr(cfg, k):
            d[k] = True
    for k in ("gloo_batch_recv", "alternate_nccl_gloo"):
        if not getattr(cfg, k):
            d[k] = False
    if cfg.activation_recompute is not None:
        d["activation_recompute"] = cfg.activation_recompute
    if cfg.schedule:
        d["schedule"] = cfg.schedule
    if cfg.activation_offload is not None:
        d["activation_offload"] = cfg.activation_offload
    if cfg.grad_norm_compat != "mean":
        d["grad_norm_compat"] = cfg.grad_norm_compat
    if cfg.comm_plan != "interleave":
        d["comm_plan"] = cfg.comm_plan
    if cfg.rank_latency_ms:
        d["rank_latency_ms"] = {str(k): v for k, v in cfg.rank_latency_ms.items()}
    if cfg.defer_tail_wgrad is not None:
        d["defer_tail_wgrad"] = cfg.defer_tail_wgrad
    d.update(cfg.extra)
    return d
