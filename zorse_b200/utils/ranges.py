"""Named ranges around engine phases: NVTX (visible to Nsight tools) and
`torch.profiler.record_function` (visible in the Chrome / TensorBoard traces the trainer
writes).  The reference only names a few FSDP-internal spans with record_function
(utils/patch.py:175-177, 694, 759, 829, 876-886); here every phase the engine issues is
named: all-gather issue / wait, reduce-scatter + Adam, optimizer, offload copies, p2p send /
receive, layer forward / backward.

Off by default (a disabled range costs one attribute test); `enable()` or ZORSE_RANGES=1
turns it on, the trainer's `--nvtx` flag does the same.
"""
from __future__ import annotations

import os

import torch

_enabled = os.environ.get("ZORSE_RANGES", "0") == "1"
_log: list | None = None   # when set (tests), range names are appended here on entry


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = on


def enabled() -> bool:
    return _enabled


def capture(log: list | None) -> None:
    """Record the names of entered ranges into `log` (None stops recording)."""
    global _log
    _log = log


class _Null:
    __slots__ = ()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NULL = _Null()


class _Range:
    __slots__ = ("name", "rf", "nvtx")

    def __init__(self, name: str):
        self.name = name
        self.rf = None
        self.nvtx = False

    def __enter__(self):
        if _log is not None:
            _log.append(self.name)
        self.rf = torch.profiler.record_function(self.name)
        self.rf.__enter__()
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
            self.nvtx = True
        return self

    def __exit__(self, *exc):
        if self.nvtx:
            torch.cuda.nvtx.range_pop()
        self.rf.__exit__(*exc)
        return False


def phase(name: str):
    """`with phase("zero.all_gather"):` — a no-op object unless ranges are enabled."""
    return _Range(name) if _enabled else _NULL
