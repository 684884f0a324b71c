"""Shared machinery of the pipeline schedules.

Every schedule exposes `step(step_idx, inputs, targets) -> loss`, the call the trainer makes
once per iteration (reference: `pp_schedule.step(...)`, zorse.py:162,
zorse_utils/pipeline_schedule_v2.py:376-409).  `inputs[g]` / `targets[g]` are the token ids
and labels of global microbatch g; a rank touches only the microbatches the static plan
gives it.  A step runs every local stage forward in ascending order, then backward in
descending order, then the optimizer (unless it already ran inside backward).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..stage import PipelineStage


class ScheduleBase:
    name = "base"
    recompute_default = True

    def __init__(self, stages: list[PipelineStage], cfg, *, recompute: Optional[bool] = None, pipeline_log=None,
                 defer_wgrad: bool = False, defer_tail_wgrad: int = 0, prepost_recv: bool = False):
        self.stages = sorted(stages, key=lambda s: s.stage_id)
        self.cfg = cfg
        # 1F1B schedules: send a microbatch's input gradient upstream before computing its weight gradients
        self.defer_wgrad = defer_wgrad
        # 1F1B, last stage: the weight gradients of the output head and of this many blocks before it run after the
        # stage's last backward, in the time the last stage otherwise idles while the other stages drain
        self.defer_tail_wgrad = int(defer_tail_wgrad)
        # 1F1B: the receive of the NEXT forward / backward is posted before the current one is computed, so the transfer
        # and its handshake run under compute (needs per-boundary process groups: `PipelineStage.split_parity`)
        self.prepost_recv = bool(prepost_recv)
        self.recompute = self.recompute_default if recompute is None else recompute
        self.log = pipeline_log
        self.device = stages[0].device if stages else torch.device("cpu")

    # -- to be provided by subclasses ----------------------------------------------
    def forward_stage(self, st: PipelineStage, inputs, targets) -> None:
        raise NotImplementedError

    def backward_stage(self, st: PipelineStage, inputs, targets) -> None:
        raise NotImplementedError

    # -- step -------------------------------------------------------------------------
    def step(self, step_idx: int, inputs, targets):
        if self.log:
            self.log.set_step(step_idx)
        for st in self.stages:
            st.loss_sum = None
        for st in self.stages:
            self.forward_stage(st, inputs, targets)
            st.flush()
        for st in reversed(self.stages):
            self.backward_stage(st, inputs, targets)
            st.flush()
        for st in self.stages:
            st.engine.optimizer_step()
            st.engine.finish_step()
            st.stash.clear()
            st.saved.clear()
        loss = None
        for st in self.stages:
            if st.is_last and st.loss_sum is not None:
                loss = st.loss_sum if loss is None else loss + st.loss_sum
        return loss

    # -- helpers ----------------------------------------------------------------------
    def _tgt(self, st: PipelineStage, targets, mbl: int):
        if not st.is_last or targets is None:
            return None
        return targets[st.microbatches[mbl]]

    def _inp(self, st: PipelineStage, inputs, mbl: int):
        return inputs[st.microbatches[mbl]]

    def _ev(self, what: str, st: PipelineStage, li: int, mbl: int):
        if self.log:
            getattr(self.log, what)(st.stage_id, li, st.microbatches[mbl])
