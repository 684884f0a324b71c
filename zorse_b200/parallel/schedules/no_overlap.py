"""Layer-major schedule without communication/compute overlap: the outputs of the last
layer are held back, the device is synchronised, and they are sent one by one, each send
waited for; gradients likewise.  Receives are posted and waited one at a time.
Reference: zorse_utils/pipeline_schedule_no_overlap.py:89-105, 184-200 (`--sync_comm`).
"""
from .layer_major import LayerMajorSchedule


class NoOverlapSchedule(LayerMajorSchedule):
    name = "no_overlap"
    recv_mode = "per_mb"
    send_mode = "deferred"
