"""Pipeline schedules and their selection by the trainer's flags
(precedence flashflex > zero2 > two-stage-sync > sync-comm > default, reference zorse.py:245-262)."""
from .base import ScheduleBase
from .flashflex import FlashflexSchedule
from .interleaved import InterleavedOneFOneBSchedule
from .layer_major import LayerMajorSchedule
from .no_overlap import NoOverlapSchedule
from .one_f_one_b import OneFOneBSchedule
from .two_stage_sync import TwoStageSyncSchedule
from .zero2 import Zero2Schedule

SCHEDULES = {
    "layer_major": LayerMajorSchedule, "default": LayerMajorSchedule, "v2": LayerMajorSchedule,
    "no_overlap": NoOverlapSchedule, "sync_comm": NoOverlapSchedule,
    "two_stage_sync": TwoStageSyncSchedule,
    "zero2": Zero2Schedule, "zero2_pipeline": Zero2Schedule,
    "flashflex": FlashflexSchedule, "flashflex_pipeline": FlashflexSchedule,
    # all forwards, then all backwards, microbatch-major with activations kept on the GPU is GPipe's order
    # (the reference names it only in its unused torch.distributed.pipelining wrapper, models/pipeline_model.py:51-78)
    "gpipe": FlashflexSchedule,
    "1f1b": OneFOneBSchedule, "one_f_one_b": OneFOneBSchedule,
    "1f1b_interleaved": InterleavedOneFOneBSchedule, "interleaved_1f1b": InterleavedOneFOneBSchedule,
}


def schedule_name_from_flags(args) -> str:
    if getattr(args, "two_stage_sync", False) and getattr(args, "sync_comm", False):
        raise ValueError("--two_stage_sync and --sync_comm cannot be combined")
    if getattr(args, "schedule", None):
        return args.schedule
    if getattr(args, "flashflex_pipeline", False):
        return "flashflex"
    if getattr(args, "zero2_pipeline", False):
        return "zero2"
    if getattr(args, "two_stage_sync", False):
        return "two_stage_sync"
    if getattr(args, "sync_comm", False):
        return "no_overlap"
    if getattr(args, "one_f_one_b", False):
        return "1f1b"
    return "layer_major"


def build_schedule(name: str, stages, cfg, **kw) -> ScheduleBase:
    if name not in SCHEDULES:
        raise ValueError(f"unknown schedule {name!r}; known: {sorted(set(SCHEDULES))}")
    cls = SCHEDULES[name]
    if not stages:
        cls = ScheduleBase                  # a rank the plan leaves idle: every step is empty
    if cls is OneFOneBSchedule and len(stages) > 1:
        cls = InterleavedOneFOneBSchedule   # several chunks per rank: the planner's interleaved plans
    return cls(stages, cfg, **kw)
