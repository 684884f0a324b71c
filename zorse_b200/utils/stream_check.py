"""Host-side race detector for stream discipline (debug mode, no device tool involved).

The engine runs collectives, p2p transfers and offload copies on side streams and hands data
between streams with events.  A missing wait is silent on the GPU (the reference has one: its
default schedule copies activations to the host on a side stream that never waited for the
compute stream, zorse_utils/pipeline_schedule_v2.py:256-262).  This module finds that class of
bug on the host: it keeps a vector clock per stream, advances and merges the clocks at every
`Event.record`, `Stream.wait_event`, `Stream.wait_stream` and synchronise call, and the engine
declares next to each cross-stream hand-off which stream last wrote a buffer (`wrote`) and which
stream is about to read it (`read`).  A read whose stream has not (transitively) waited for the
writer is recorded as a violation and, with `strict`, raises.

`install()` patches the torch.cuda stream / event methods so that ordinary engine code is
tracked without changes; the logic itself (`StreamOrderChecker`) works on any hashable stream
ids and is unit-tested on CPU.  Off by default: every hook is one `is None` test.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Hashable, Optional


class StreamOrderError(RuntimeError):
    pass


@dataclass
class Violation:
    key: Hashable
    reader: Hashable
    writer: Hashable
    label: str

    def __str__(self):
        return (f"buffer {self.key!r}: stream {self.reader!r} reads ({self.label}) without having waited for the "
                f"write on stream {self.writer!r}")


class StreamOrderChecker:
    def __init__(self, strict: bool = False):
        self.strict = strict
        self.vc: dict = {}        # stream -> {stream: tick}
        self.events: dict = {}    # event id -> snapshot of the recording stream's clock
        self.writes: dict = {}    # buffer key -> (stream, tick)
        self.violations: list[Violation] = []
        self.checked = 0

    # -- clocks -----------------------------------------------------------------------
    def _clock(self, s) -> dict:
        c = self.vc.get(s)
        if c is None:
            c = self.vc[s] = {s: 0}
        return c

    def _tick(self, s) -> int:
        c = self._clock(s)
        c[s] += 1
        return c[s]

    @staticmethod
    def _merge(dst: dict, src: dict) -> None:
        for k, v in src.items():
            if dst.get(k, 0) < v:
                dst[k] = v

    def record(self, event: Hashable, stream) -> None:
        self._tick(stream)
        self.events[event] = dict(self._clock(stream))

    def wait_event(self, stream, event: Hashable) -> None:
        snap = self.events.get(event)
        if snap is not None:
            self._merge(self._clock(stream), snap)

    def wait_stream(self, stream, other) -> None:
        if stream == other:
            return
        self._tick(other)
        self._merge(self._clock(stream), self._clock(other))

    def synchronize(self, stream=None) -> None:
        """Host waited for `stream` (or the whole device): what ran there is visible to every
        stream from now on (anything issued later is ordered after the host wait)."""
        srcs = [stream] if stream is not None else list(self.vc)
        for s in srcs:
            for c in self.vc.values():
                self._merge(c, self._clock(s))

    def event_synchronize(self, event: Hashable) -> None:
        snap = self.events.get(event)
        if snap is not None:
            for c in self.vc.values():
                self._merge(c, snap)

    # -- declarations -------------------------------------------------------------------
    def wrote(self, key: Hashable, stream) -> None:
        self.writes[key] = (stream, self._tick(stream))

    def read(self, key: Hashable, stream, label: str = "") -> bool:
        w = self.writes.get(key)
        if w is None:
            return True
        self.checked += 1
        ws, tick = w
        if ws == stream or self._clock(stream).get(ws, 0) >= tick:
            return True
        v = Violation(key, stream, ws, label)
        self.violations.append(v)
        if self.strict:
            raise StreamOrderError(str(v))
        return False

    def forget(self, key: Hashable) -> None:
        self.writes.pop(key, None)

    def report(self) -> str:
        if not self.violations:
            return f"stream order: {self.checked} cross-stream reads checked, no violation"
        return "\n".join([f"stream order: {len(self.violations)} violation(s) in {self.checked} checked reads"] +
                         [f"  {v}" for v in self.violations[:20]])


# ---------------------------------------------------------------------------------------
# process-wide instance + hooks used by the engine
# ---------------------------------------------------------------------------------------
_active: Optional[StreamOrderChecker] = None
_patched = False


def active() -> Optional[StreamOrderChecker]:
    return _active


def _sid(stream) -> Hashable:
    return getattr(stream, "cuda_stream", stream)


def _current():
    import torch

    return torch.cuda.current_stream().cuda_stream


def wrote(key: Hashable, stream=None) -> None:
    """`stream` (default: the current CUDA stream) has just been given work that writes `key`."""
    if _active is None:
        return
    _active.wrote(key, _current() if stream is None else _sid(stream))


def read(key: Hashable, stream=None, label: str = "") -> None:
    """`stream` (default: current) is about to be given work that reads `key`."""
    if _active is None:
        return
    _active.read(key, _current() if stream is None else _sid(stream), label)


def install(strict: bool = False) -> StreamOrderChecker:
    """Activates the checker and (once) wraps the torch.cuda stream / event methods."""
    global _active, _patched
    _active = StreamOrderChecker(strict)
    if _patched:
        return _active
    import torch

    S, E = torch.cuda.Stream, torch.cuda.Event
    o_we, o_ws, o_ss, o_re = S.wait_event, S.wait_stream, S.synchronize, S.record_event
    o_er, o_ew, o_es = E.record, E.wait, E.synchronize
    o_sync = torch.cuda.synchronize

    def wait_event(self, event):
        if _active is not None:
            _active.wait_event(self.cuda_stream, id(event))
        return o_we(self, event)

    def wait_stream(self, stream):
        if _active is not None:
            _active.wait_stream(self.cuda_stream, stream.cuda_stream)
        return o_ws(self, stream)

    def stream_sync(self):
        r = o_ss(self)
        if _active is not None:
            _active.synchronize(self.cuda_stream)
        return r

    def record_event(self, event=None):
        ev = o_re(self, event)
        if _active is not None:
            _active.record(id(ev), self.cuda_stream)
        return ev

    def ev_record(self, stream=None):
        r = o_er(self, stream) if stream is not None else o_er(self)
        if _active is not None:
            _active.record(id(self), _current() if stream is None else stream.cuda_stream)
        return r

    def ev_wait(self, stream=None):
        if _active is not None:
            _active.wait_event(_current() if stream is None else stream.cuda_stream, id(self))
        return o_ew(self, stream) if stream is not None else o_ew(self)

    def ev_sync(self):
        r = o_es(self)
        if _active is not None:
            _active.event_synchronize(id(self))
        return r

    def dev_sync(device=None):
        r = o_sync(device)
        if _active is not None:
            _active.synchronize()
        return r

    S.wait_event, S.wait_stream, S.synchronize, S.record_event = wait_event, wait_stream, stream_sync, record_event
    E.record, E.wait, E.synchronize = ev_record, ev_wait, ev_sync
    torch.cuda.synchronize = dev_sync
    _patched = True
    return _active


def uninstall() -> None:
    """Stops checking (the wrappers stay in place and become pass-throughs)."""
    global _active
    _active = None
