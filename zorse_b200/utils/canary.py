"""Canary words around buffers that kernels and copy engines write through raw pointers
(symmetric-memory parameter / gradient buffers, pinned staging buffers).  Debug aid: with
ZORSE_DEBUG_CANARY=1 such buffers are allocated with a guard band of a known bit pattern on
both sides and `check_all()` (called by the trainer after every step) reports any band that
changed, i.e. an out-of-bounds write, with the buffer's label.  Off by default: `guarded`
then returns the plain allocation.  The reference has no counterpart.
"""
from __future__ import annotations

import os
from typing import Callable

import torch

GUARD_BYTES = 256
PATTERN = 0x5A


def enabled() -> bool:
    return os.environ.get("ZORSE_DEBUG_CANARY", "0") == "1"


class CanaryError(RuntimeError):
    pass


_registry: list = []   # (label, raw uint8 view, payload bytes)


def guard_elems(dtype: torch.dtype) -> int:
    """Guard elements per side for `dtype` (whole elements, so the payload keeps its alignment)."""
    esz = torch.empty((), dtype=dtype).element_size()
    return (GUARD_BYTES + esz - 1) // esz


def register(label: str, raw: torch.Tensor, numel: int) -> torch.Tensor:
    """`raw` holds numel + 2 * guard_elems(dtype) elements: fills both bands, remembers the buffer
    and returns the payload view."""
    g = guard_elems(raw.dtype)
    assert raw.numel() == numel + 2 * g and raw.is_contiguous()
    esz = raw.element_size()
    b = raw.view(torch.uint8)
    b[: g * esz] = PATTERN
    b[(g + numel) * esz:] = PATTERN
    _registry.append((label, b, g * esz, numel * esz))
    return raw[g:g + numel]


def guarded(numel: int, dtype: torch.dtype, alloc: Callable[[int, torch.dtype], torch.Tensor], label: str,
            force: bool = False) -> torch.Tensor:
    """Returns a `numel`-element tensor of `dtype` from `alloc(n, dtype)`.  In canary mode the
    allocation is GUARD_BYTES larger on each side and the bands are filled with PATTERN."""
    if not (force or enabled()):
        return alloc(numel, dtype)
    return register(label, alloc(numel + 2 * guard_elems(dtype), dtype), numel)


def check_all(raise_on_error: bool = True) -> list[str]:
    """Names of the buffers whose guard bands were overwritten."""
    bad = []
    for label, b, gbytes, payload in _registry:
        lo, hi = b[:gbytes], b[gbytes + payload:]
        if not (bool((lo == PATTERN).all()) and bool((hi == PATTERN).all())):
            side = "before" if not bool((lo == PATTERN).all()) else "after"
            bad.append(f"{label} (band {side} the buffer)")
    if bad and raise_on_error:
        raise CanaryError("out-of-bounds write detected next to: " + "; ".join(bad))
    return bad


def reset() -> None:
    _registry.clear()
