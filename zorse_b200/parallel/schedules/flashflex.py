"""Flashflex-style schedule: the ZeRO-2 pipeline schedule with layer inputs kept on the GPU
(no host offload of activations) and no batched stage sync.  Layers are still recomputed
in backward.  Reference: zorse_utils/pipeline_schedule_flashflex.py:229-503
(`--flashflex_pipeline`).
"""
from .zero2 import Zero2Schedule


class FlashflexSchedule(Zero2Schedule):
    name = "flashflex"

    def __init__(self, stages, cfg, **kw):
        super().__init__(stages, cfg, **kw)
        self.deferred_sends = False
        for st in self.stages:
            st.stash.offload = False
