"""Interleaved 1F1B: every rank hosts v model chunks (stages g, g + P, g + 2P, ... of a
pipeline of P rank groups), which divides the pipeline bubble by v at the price of v times as
many boundary transfers.

The reference only has the dormant torch.distributed.pipelining wrapper for this
(models/pipeline_model.py:51-78, `ScheduleInterleaved1F1B`); its live interleaving
(zorse_optimizer/optimizer.py:200-280) runs each local stage all-forward-then-all-backward.
Here the order is the usual one for interleaved 1F1B: virtual step k runs chunk
`(k mod P v) div P` (mirrored for backward) on microbatch `(k div P v) P + k mod P`, a warm-up of
`2 (P - g - 1) + (v - 1) P` forwards, then one forward / one backward per step, then the
remaining backwards.  Parameters stay unsharded for the step, activations are kept.

Needs the same number of microbatches per rank on every stage of a rank and that number to be a
multiple of P.  Receives are posted when needed (see one_f_one_b.py for why).
"""
from __future__ import annotations

from .base import ScheduleBase


class InterleavedOneFOneBSchedule(ScheduleBase):
    name = "1f1b_interleaved"
    recompute_default = False

    def step(self, step_idx, inputs, targets):
        if self.log:
            self.log.set_step(step_idx)
        sts = self.stages                       # this rank's chunks, ascending stage order
        v = len(sts)
        order = [s.stage_id for s in self.cfg.stages]
        if len(order) % v:
            raise ValueError("interleaved 1F1B: every rank group must host the same number of stages")
        P = len(order) // v
        pos = [order.index(s.stage_id) for s in sts]
        g = pos[0]
        if g >= P or any(pos[c] != g + c * P for c in range(v)):
            raise ValueError(f"interleaved 1F1B: stages {pos} of this rank are not g, g+P, g+2P, ... with P = {P}")
        M = sts[0].M
        if any(s.M != M or s.microbatches != sts[0].microbatches for s in sts):
            raise ValueError("interleaved 1F1B: the stages of a rank must own the same microbatches")
        if M % P:
            raise ValueError(f"interleaved 1F1B: {M} microbatches per rank is not a multiple of {P} rank groups")
        for st in sts:
            st.loss_sum = None
            st.engine.prefetch_all()
        T = M * v
        warm = min(2 * (P - g - 1) + (v - 1) * P, T)

        def chunk_of(k, forward):
            c = (k % (P * v)) // P
            return c if forward else v - 1 - c

        def mb_of(k):
            return (k // (P * v)) * P + k % P

        def fwd(k):
            st, mbl = sts[chunk_of(k, True)], mb_of(k)
            units = st.engine.units
            x = self._inp(st, inputs, mbl) if st.is_first else st.recv_fwd(mbl).wait()
            for li in range(len(st.layers)):
                units[li].acquire()
                x = st.forward_layer(li, mbl, x, self._tgt(st, targets, mbl), self.recompute)
            if not st.is_last:
                st.send_fwd(mbl, x)

        def bwd(k):
            st, mbl = sts[chunk_of(k, False)], mb_of(k)
            units = st.engine.units
            dy = None if st.is_last else st.recv_bwd(mbl).wait()
            last, asynchronous = mbl == M - 1, st.device.type == "cuda"   # see one_f_one_b.py
            defer = self.defer_wgrad and not last and not st.is_first and st.can_defer_wgrad()
            st.wgrad.active = defer
            for li in reversed(range(len(st.layers))):
                units[li].acquire()
                units[li].grad_views()
                dy = st.backward_layer(li, mbl, dy, self._tgt(st, targets, mbl), self.recompute)
                if last and asynchronous:
                    units[li].reduce_grads()
            if not st.is_first:
                st.send_bwd(mbl, dy)
            if defer:
                st.wgrad.active = False
                st.wgrad.flush()
            if last and not asynchronous:
                for li in reversed(range(len(st.layers))):
                    units[li].reduce_grads()

        for k in range(warm):
            fwd(k)
        for k in range(T - warm):
            fwd(warm + k)
            bwd(k)
        for k in range(T - warm, T):
            bwd(k)
        if M == 0:
            # no microbatches: join the reductions in the order the peers reach them (chunks from the
            # last to the first, layers from the last to the first)
            for st in reversed(sts):
                for u in reversed(st.engine.units):
                    u.grad_views()
                    u.reduce_grads()
        loss = None
        for st in sts:
            st.flush()
            st.engine.optimizer_step()
            st.engine.finish_step()
            st.stash.clear()
            st.saved.clear()
            if st.is_last and st.loss_sum is not None:
                loss = st.loss_sum if loss is None else loss + st.loss_sum
        return loss
