"""Default schedule: layer-major execution ("for layer: for microbatch").

Each layer's parameters are gathered once per pass and its gradients reduced once per
step whatever the number of microbatches; only layer-boundary activations are kept and
every layer is recomputed in backward.  This is the reference's default schedule
(zorse_utils/pipeline_schedule_v2.py:202-374); the communication variants of
`no_overlap.py` and `two_stage_sync.py` are the same loop with different send / receive
timing, selected by `recv_mode` and `send_mode`.
"""
from __future__ import annotations

import torch

from ..stage import PipelineStage
from .base import ScheduleBase


class LayerMajorSchedule(ScheduleBase):
    name = "layer_major"
    recompute_default = True
    # "prepost": post every receive of the pass up front, wait per microbatch
    # "per_mb":  post and wait one receive at a time
    # "upfront": post and wait for every receive before computing
    recv_mode = "prepost"
    # "per_mb": send as soon as a microbatch leaves the last layer
    # "deferred": keep outputs, synchronise the device, then send one by one, waiting on each
    send_mode = "per_mb"

    def modes(self, st: PipelineStage):
        return self.recv_mode, self.send_mode

    def _recv_all(self, st, fn, order, mode):
        if mode == "per_mb":
            return {}
        hs = {mbl: fn(mbl) for mbl in order}
        if mode == "upfront":
            for h in hs.values():
                h.wait()
        return hs

    def _send_deferred(self, st, fn, items):
        if st.device.type == "cuda":
            torch.cuda.synchronize()
        for mbl, t in items:
            fn(mbl, t).wait()

    def forward_stage(self, st: PipelineStage, inputs, targets):
        L, M = len(st.layers), st.M
        recv_mode, send_mode = self.modes(st)
        units = st.engine.units
        last_local = st is self.stages[-1]
        outs = {}
        handles = {} if st.is_first else self._recv_all(st, st.recv_fwd, range(M), recv_mode)
        for li in range(L):
            units[li].acquire()
            if li + 1 < L:
                units[li + 1].prefetch()
            deferred = []
            for mbl in range(M):
                if li == 0:
                    if st.is_first:
                        x = self._inp(st, inputs, mbl)
                    else:
                        self._ev("log_forward_recv", st, li, mbl)
                        x = (handles.pop(mbl) if mbl in handles else st.recv_fwd(mbl)).wait()
                else:
                    x = outs.pop(mbl)
                self._ev("log_forward_compute", st, li, mbl)
                y = st.forward_layer(li, mbl, x, self._tgt(st, targets, mbl), self.recompute)
                if li == L - 1:
                    if not st.is_last:
                        if send_mode == "per_mb":
                            self._ev("log_forward_send", st, li, mbl)
                            st.send_fwd(mbl, y)
                        else:
                            deferred.append((mbl, y))
                else:
                    outs[mbl] = y
            if deferred:
                self._send_deferred(st, st.send_fwd, deferred)
            # keep the last layer of the rank's last stage: backward starts with it
            if not (last_local and li == L - 1):
                units[li].release()

    def backward_stage(self, st: PipelineStage, inputs, targets):
        L, M = len(st.layers), st.M
        recv_mode, send_mode = self.modes(st)
        units = st.engine.units
        grads = {}
        handles = {} if st.is_last else self._recv_all(st, st.recv_bwd, reversed(range(M)), recv_mode)
        for li in reversed(range(L)):
            units[li].acquire()
            if li > 0:
                units[li - 1].prefetch()
            units[li].grad_views()
            deferred = []
            for mbl in reversed(range(M)):
                if li == L - 1:
                    if st.is_last:
                        dy = None
                    else:
                        self._ev("log_backward_recv", st, li, mbl)
                        dy = (handles.pop(mbl) if mbl in handles else st.recv_bwd(mbl)).wait()
                else:
                    dy = grads.pop(mbl)
                self._ev("log_backward_compute", st, li, mbl)
                dx = st.backward_layer(li, mbl, dy, self._tgt(st, targets, mbl), self.recompute)
                if li == 0:
                    if not st.is_first:
                        if send_mode == "per_mb":
                            self._ev("log_backward_send", st, li, mbl)
                            st.send_bwd(mbl, dx)
                        else:
                            deferred.append((mbl, dx))
                else:
                    grads[mbl] = dx
            if deferred:
                self._send_deferred(st, st.send_bwd, deferred)
            units[li].reduce_grads()
            units[li].release()
