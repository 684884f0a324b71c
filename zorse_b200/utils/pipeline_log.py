"""Per-rank pipeline event log `./zorse_logs/pipeline_rank_<r>.log`: one line per receive /
compute / send of every (stage, layer, microbatch), for checking the order of events
(reference zorse_utils/pipeline_logger.py:21-133)."""
from __future__ import annotations

import logging
import os

_instance = None


class PipelineLogger:
    def __init__(self, log_dir: str = "./zorse_logs", rank: int = 0, level: str = "INFO"):
        os.makedirs(log_dir, exist_ok=True)
        self.path = os.path.join(log_dir, f"pipeline_rank_{rank}.log")
        self.log = logging.getLogger(f"zorse.pipeline.{rank}")
        self.log.handlers.clear()
        h = logging.FileHandler(self.path, mode="w")
        h.setFormatter(logging.Formatter("%(asctime)s %(message)s"))
        self.log.addHandler(h)
        self.log.setLevel(getattr(logging, level.upper(), logging.INFO))
        self.log.propagate = False
        self.step = 0
        self.events: list = []

    def set_step(self, step: int):
        self.step = step

    def _e(self, what, stage, layer, mb):
        self.events.append((self.step, what, stage, layer, mb))
        self.log.info(f"step={self.step} {what} stage={stage} layer={layer} microbatch={mb}")

    def log_forward_recv(self, s, l, m): self._e("fwd_recv", s, l, m)
    def log_forward_compute(self, s, l, m): self._e("fwd_compute", s, l, m)
    def log_forward_send(self, s, l, m): self._e("fwd_send", s, l, m)
    def log_backward_recv(self, s, l, m): self._e("bwd_recv", s, l, m)
    def log_backward_compute(self, s, l, m): self._e("bwd_compute", s, l, m)
    def log_backward_send(self, s, l, m): self._e("bwd_send", s, l, m)


def init_pipeline_logger(log_dir: str = "./zorse_logs", rank: int = 0, level: str = "INFO") -> PipelineLogger:
    global _instance
    _instance = PipelineLogger(log_dir, rank, level)
    return _instance


def get_pipeline_logger():
    return _instance
