"""Two GPU groups alternating stages never send to each other at the same time.

Even stages receive everything up front and send per microbatch; odd stages receive per
microbatch and send everything after a device synchronisation; mirrored for gradients.
Reference: zorse_utils/pipeline_schedule_two_stage_sync.py:1-19, 56-171 (`--two_stage_sync`).
"""
from .layer_major import LayerMajorSchedule


class TwoStageSyncSchedule(LayerMajorSchedule):
    name = "two_stage_sync"

    def modes(self, st):
        if st.stage_id % 2 == 0:
            return "upfront", "per_mb"
        return "per_mb", "deferred"
