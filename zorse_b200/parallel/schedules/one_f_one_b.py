"""True 1F1B: warm-up forwards, steady one-forward-one-backward, cool-down backwards.

The reference ships no 1F1B on its live path (its schedules are all-forward-then-all-backward,
zorse_utils/pipeline_schedule_v2.py:391-402; "1f1b" only names a dormant
torch.distributed.pipelining wrapper, models/pipeline_model.py:51-78).  Parameters stay
unsharded for the whole step (gathered once), gradients are reduced after a layer's last
backward microbatch.  By default activations are kept (no recompute): at most
`num_stages - stage_index` microbatches are in flight per rank.
"""
from __future__ import annotations

from ..p2p_plan import is_regular, plan_1f1b_order
from .base import ScheduleBase


class OneFOneBSchedule(ScheduleBase):
    name = "1f1b"
    recompute_default = False

    def __init__(self, stages, cfg, **kw):
        super().__init__(stages, cfg, **kw)
        # mixed stage widths or uneven microbatch counts: the classic warm-up / alternate / drain
        # order can deadlock there (see p2p_plan.plan_1f1b_order), so take the order from the plan
        self.order = None
        if len(self.stages) == 1 and not is_regular(cfg):
            self.order = plan_1f1b_order(cfg)[self.stages[0].rank]

    def step(self, step_idx, inputs, targets):
        if len(self.stages) != 1:
            raise ValueError("the 1F1B schedule runs one stage per rank (no interleaving)")
        if self.log:
            self.log.set_step(step_idx)
        st = self.stages[0]
        st.loss_sum = None
        L, M = len(st.layers), st.M
        units = st.engine.units
        st.engine.prefetch_all()
        stage_pos = [s.stage_id for s in self.cfg.stages].index(st.stage_id)
        warm = min(len(self.cfg.stages) - stage_pos - 1, M)
        # The last stage carries the output head on top of its blocks, so it sets the pipeline's period, and it
        # is also the stage that idles longest at the end of a step (while the other stages drain).  With
        # `defer_tail_wgrad = k` the weight-gradient GEMMs of its last k layers (the head first) are taken out of
        # every microbatch's backward and run once, after the stage's last backward, inside that idle time.  The
        # operands (dlogits, layer inputs) of all microbatches stay alive until then.  Same additions in the same
        # order per bucket entry, so the result is bit-identical.  Whether it pays is the caller's question
        # (`planner.predict.best_tail_deferral`): the held-back work has to fit into the time the other stages
        # need to drain, and with one stage there is nothing to gain.
        hold = set()
        if self.defer_tail_wgrad > 0 and st.is_last and st.can_defer_wgrad():
            hold = set(range(max(L - self.defer_tail_wgrad, 0), L))
        # By default receives are posted when they are needed, never ahead: torch serialises the p2p
        # operations of one process group on each rank, so a receive posted one microbatch early
        # would sit in front of this rank's own send of the current microbatch, and across four
        # or more stages those extra "send waits for the next receive" edges close a cycle
        # (stage 0's first backward would wait for a forward it runs only afterwards).
        # `prepost_recv` posts the receive of the next operation (one operation ahead, not one microbatch) before
        # the current one is computed.  It is only allowed with per-boundary groups (the stage's `split_parity`),
        # where a group carries one direction of one boundary on a rank, so that by construction an early receive
        # stands in front of nothing but later receives of that boundary; the host-side replay checks the program
        # all the same before a job starts.
        if self.prepost_recv and not st.split_parity:
            raise ValueError("prepost_recv needs per-boundary process groups (PipelineStage(split_parity=True))")
        posted: dict = {}

        def post(op, mbl):
            # the receive operation `op` on microbatch `mbl` will wait for, if it has one and it is not posted yet
            if (op, mbl) in posted or (st.is_first if op == "F" else st.is_last):
                return
            posted[(op, mbl)] = st.recv_fwd(mbl) if op == "F" else st.recv_bwd(mbl)

        def take(op, mbl):
            post(op, mbl)
            return posted.pop((op, mbl)).wait()

        def fwd(mbl):
            x = self._inp(st, inputs, mbl) if st.is_first else take("F", mbl)
            for li in range(L):
                units[li].acquire()
                x = st.forward_layer(li, mbl, x, self._tgt(st, targets, mbl), self.recompute)
            if not st.is_last:
                st.send_fwd(mbl, x)

        def bwd(mbl):
            dy = None if st.is_last else take("B", mbl)
            # On CUDA the reduction of a layer is queued on the communication stream as soon as its last
            # backward is issued and overlaps the rest of that backward.  Host-blocking collectives (gloo)
            # must wait until this microbatch's gradient has been sent upstream: a rank that finishes early
            # would otherwise sit in the collective while upstream stages still need that gradient to
            # produce the forwards its peers are waiting for.
            last, asynchronous = mbl == M - 1, st.device.type == "cuda"
            # weight gradients after the send (not for the last microbatch, whose layers are reduced as they finish)
            defer = self.defer_wgrad and not last and not st.is_first and st.can_defer_wgrad()
            st.wgrad.active = defer
            for li in reversed(range(L)):
                units[li].acquire()
                units[li].grad_views()
                dy = st.backward_layer(li, mbl, dy, self._tgt(st, targets, mbl), self.recompute, hold_wgrad=li in hold)
                if last and asynchronous and li not in hold:
                    units[li].reduce_grads()
            if not st.is_first:
                st.send_bwd(mbl, dy)
            if defer:
                st.wgrad.active = False
                st.wgrad.flush()
            if last and not asynchronous:
                for li in reversed(range(L)):
                    if li not in hold:
                        units[li].reduce_grads()

        if self.order is not None:
            seq = list(self.order)
        else:
            seq = [("F", i) for i in range(warm)]
            for i in range(M - warm):
                seq += [("F", warm + i), ("B", i)]
            seq += [("B", i) for i in range(M - warm, M)]
        for j, (op, i) in enumerate(seq):
            if self.prepost_recv:
                post(op, i)
                if j + 1 < len(seq):
                    post(*seq[j + 1])
            (fwd if op == "F" else bwd)(i)
        if hold and M > 0:
            # the held-back weight gradients, then the reductions of the layers they belong to (last layer first,
            # the order every rank of the stage uses)
            st.wgrad_tail.active = False
            st.wgrad_tail.flush()
            for li in sorted(hold, reverse=True):
                units[li].acquire()
                units[li].grad_views()
                units[li].reduce_grads()
        if M == 0:
            # a rank without microbatches still joins every reduction, in the order its peers use
            # (last layer first; layers whose weight gradients are held back come after the others)
            for li in [i for i in reversed(range(L)) if i not in hold] + sorted(hold, reverse=True):
                units[li].grad_views()
                units[li].reduce_grads()
        st.flush()
        st.engine.optimizer_step()
        st.engine.finish_step()
        st.stash.clear()
        st.saved.clear()
        return st.loss_sum if st.is_last else None
