"""ZeRO-2 pipeline schedule: microbatch-major ("for microbatch: for layer").

The whole stage is unsharded ahead of use (prefetch of every layer), the rank's last local
stage stays unsharded from forward through backward, earlier local stages are freed after
their forward and gathered again, in reverse layer order, before their backward; the next
microbatch's receive is posted one microbatch ahead; gradients are reduce-scattered once
per layer after its last microbatch.  Layer-boundary activations are stashed (optionally
in pinned host memory) and layers are recomputed in backward.
Reference: zorse_utils/pipeline_schedule_zero2.py:220-633 (`--zero2_pipeline`).
`interleave_stage_sync` (sends held back and issued together after a device sync),
`gloo_batch_recv` (all Gloo receives of a pass posted up front) and `alternate_nccl_gloo`
(NCCL on equal-width boundaries, Gloo on mixed-width ones) are honoured.
"""
from __future__ import annotations

import torch

from ..stage import PipelineStage
from .base import ScheduleBase


class Zero2Schedule(ScheduleBase):
    name = "zero2"
    recompute_default = True

    def __init__(self, stages, cfg, **kw):
        super().__init__(stages, cfg, **kw)
        self.deferred_sends = bool(getattr(cfg, "interleave_stage_sync", False))

    def forward_stage(self, st: PipelineStage, inputs, targets):
        L, M = len(st.layers), st.M
        units = st.engine.units
        st.engine.prefetch_all()
        # Gloo receives are tagged and order-free: with gloo_batch_recv all of them are posted now
        batch = (not st.is_first) and st.uses_gloo(False) and self.cfg.gloo_batch_recv
        posted = {m: st.recv_fwd(m) for m in range(M)} if batch else {}
        nxt = st.recv_fwd(0) if (not st.is_first and M > 0 and not batch) else None
        held = []
        for mbl in range(M):
            if st.is_first:
                x = self._inp(st, inputs, mbl)
            else:
                self._ev("log_forward_recv", st, 0, mbl)
                x = (posted.pop(mbl) if batch else nxt).wait()
                nxt = None
            for li in range(L):
                units[li].acquire()
                self._ev("log_forward_compute", st, li, mbl)
                x = st.forward_layer(li, mbl, x, self._tgt(st, targets, mbl), self.recompute)
                if li == 0 and not st.is_first and mbl + 1 < M and not batch:
                    nxt = st.recv_fwd(mbl + 1)  # one-ahead receive
            if not st.is_last:
                if self.deferred_sends:
                    held.append((mbl, x))
                else:
                    self._ev("log_forward_send", st, L - 1, mbl)
                    st.send_fwd(mbl, x)
        if held:
            if st.device.type == "cuda":
                torch.cuda.synchronize()
            for mbl, y in held:
                st.send_fwd(mbl, y)
        if st is not self.stages[-1]:
            for u in units:
                u.release(force=True)

    def backward_stage(self, st: PipelineStage, inputs, targets):
        L, M = len(st.layers), st.M
        units = st.engine.units
        st.engine.prefetch_all(reverse=True)
        batch = (not st.is_last) and st.uses_gloo(True) and self.cfg.gloo_batch_recv
        posted = {m: st.recv_bwd(m) for m in range(M)} if batch else {}
        nxt = st.recv_bwd(M - 1) if (not st.is_last and M > 0 and not batch) else None
        held = []
        for mbl in reversed(range(M)):
            if st.is_last:
                dy = None
            else:
                self._ev("log_backward_recv", st, L - 1, mbl)
                dy = (posted.pop(mbl) if batch else nxt).wait()
                nxt = None
            for li in reversed(range(L)):
                units[li].acquire()
                units[li].grad_views()
                self._ev("log_backward_compute", st, li, mbl)
                dy = st.backward_layer(li, mbl, dy, self._tgt(st, targets, mbl), self.recompute)
                if li == L - 1 and not st.is_last and mbl > 0 and not batch:
                    nxt = st.recv_bwd(mbl - 1)
                if mbl == 0:
                    units[li].reduce_grads()
            if not st.is_first:
                if self.deferred_sends:
                    held.append((mbl, dy))
                else:
                    self._ev("log_backward_send", st, 0, mbl)
                    st.send_bwd(mbl, dy)
        if M == 0:
            # a rank without microbatches still joins every reduction, in the order its peers use
            # (last layer first)
            for u in reversed(units):
                u.grad_views()
                u.reduce_grads()
        if held:
            if st.device.type == "cuda":
                torch.cuda.synchronize()
            for mbl, d in held:
                st.send_bwd(mbl, d)
