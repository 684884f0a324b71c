"""Failure detection on the host: per-step heartbeats and a watchdog.

The reference has none (only collective timeouts, utils/comm.py:15, 113-114).  Here every
rank publishes `(step, wall time)` to the rendezvous store after each step; `stale_ranks`
names ranks whose heartbeat is older than a limit, and `Watchdog` is a thread that turns a
step that exceeds its time limit into a diagnostic dump and a clean abort (`os._exit`)
instead of a silent hang.  Device-side waits are bounded separately (kernel status word).
Nothing here touches a GPU.
"""
from __future__ import annotations

import faulthandler
import os
import sys
import threading
import time
from typing import Callable, Optional


class Heartbeat:
    """Writes `hb/<rank>` = "step:time" into a key-value store (torch TCPStore/FileStore or any
    object with set/get)."""

    def __init__(self, store, rank: int, world: int, clock: Callable[[], float] = time.time):
        self.store, self.rank, self.world, self.clock = store, rank, world, clock

    def beat(self, step: int) -> None:
        """Step `step` is finished on this rank."""
        self.store.set(f"hb/{self.rank}", f"{step}:{self.clock():.3f}")

    def beat_enter(self, step: int) -> None:
        """This rank is about to run step `step`.  When a job stops, every rank that waits for a stuck peer has
        finished the same step as that peer; what tells them apart is that they have entered the next one."""
        self.store.set(f"hbin/{self.rank}", f"{step}:{self.clock():.3f}")

    def not_entered(self, step: int) -> list[int]:
        """Ranks that have not reported entering step `step` (or any later one)."""
        out = []
        for r in range(self.world):
            hb = self.read(r, key="hbin")
            if hb is None or hb[0] < step:
                out.append(r)
        return out

    def read(self, rank: int, key: str = "hb"):
        try:
            check = getattr(self.store, "check", None)     # TCPStore.get blocks on a missing key
            if check is not None and not check([f"{key}/{rank}"]):
                return None
            v = self.store.get(f"{key}/{rank}")
        except (KeyError, RuntimeError, TimeoutError):   # key never written / store gone
            return None
        if isinstance(v, bytes):
            v = v.decode()
        if not v:
            return None
        try:                                  # a short or garbled read counts as no heartbeat, not as a crash
            s, t = v.split(":")
            return int(s), float(t)
        except ValueError:
            return None

    def stale_ranks(self, limit_s: float, min_step: Optional[int] = None) -> list[int]:
        """Ranks with no heartbeat, one older than limit_s, or (if given) behind min_step."""
        now, out = self.clock(), []
        for r in range(self.world):
            hb = self.read(r)
            if hb is None or now - hb[1] > limit_s or (min_step is not None and hb[0] < min_step):
                out.append(r)
        return out


class DictStore:
    """In-process stand-in for a rendezvous store (tests)."""

    def __init__(self):
        self.d: dict = {}

    def set(self, k, v):
        self.d[k] = v

    def get(self, k):
        return self.d.get(k, "")


class Watchdog(threading.Thread):
    def __init__(self, timeout_s: float, rank: int = 0, on_timeout: Optional[Callable[[int, float], None]] = None,
                 poll_s: float = 0.5, startup_s: Optional[float] = None):
        """`startup_s`: limit that applies until the first beat (the first step pays for lazy communicator
        set-up, library loading and allocator warm-up, several times a normal step); default: timeout_s."""
        super().__init__(daemon=True)
        self.timeout_s, self.rank, self.poll_s = timeout_s, rank, poll_s
        self.startup_s = max(timeout_s, startup_s) if startup_s is not None else timeout_s
        self.on_timeout = on_timeout or self._abort
        self._last = time.monotonic()
        self._step = -1
        self._stop = threading.Event()
        self.fired = False

    def beat(self, step: int) -> None:
        self._step = step
        self._last = time.monotonic()

    def stop(self) -> None:
        self._stop.set()

    def run(self) -> None:
        while not self._stop.wait(self.poll_s):
            idle = time.monotonic() - self._last
            if idle > (self.startup_s if self._step < 0 else self.timeout_s):
                self.fired = True
                self.on_timeout(self._step, idle)
                return

    def _abort(self, step: int, idle: float) -> None:
        sys.stderr.write(f"[watchdog] rank {self.rank}: no progress for {idle:.1f}s after step {step}; "
                         f"dumping stacks and aborting\n")
        faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
        sys.stderr.flush()
        os._exit(3)


def tcp_heartbeat(rank: int, world: int, port_offset: int = 23, timeout_s: float = 60.0) -> Optional[Heartbeat]:
    """Heartbeat over a TCPStore next to the rendezvous port (rank 0 hosts it). None for one rank."""
    if world <= 1:
        return None
    import datetime

    from torch.distributed import TCPStore

    host = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + port_offset
    store = TCPStore(host, port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=timeout_s),
                     wait_for_workers=False)
    return Heartbeat(store, rank, world)


def parse_fault(spec: Optional[str]):
    """`rank:step:kind` with kind in stall | raise | exit | drop | delay=<seconds> -> (rank, step, kind); host-side
    fault injection for failure-detection tests (nothing on the device is made to fault).  `drop` loses the rank's
    first pipeline message of that step, `delay=<s>` holds it back for s seconds (both need the trainer's
    `p2p_fault_hooks`)."""
    if not spec:
        return None
    r, s, kind = spec.split(":")
    if kind not in ("stall", "raise", "exit", "drop") and not kind.startswith("delay="):
        raise ValueError(f"unknown fault kind {kind!r}")
    if kind.startswith("delay="):
        float(kind[6:])
    return int(r), int(s), kind


def injection_refusal(on_cuda: bool, collectives: str, env=None) -> Optional[str]:
    """Why host-side fault injection must not run with this set-up, or None if it may.

    A rank that leaves the job while its device memory is bound to an NVLink multicast object
    raises NVLink faults on the GPUs of the ranks that stay.  Memory gets bound that way by NCCL's
    NVLS algorithms (on by default on NVSwitch systems) and by the symmetric-memory buffers of the
    fused collectives (`multimem` variants of the fused reduce-scatter + Adam).  So on CUDA devices
    injection is only allowed when NCCL_NVLS_ENABLE=0 was set before start-up, the collectives are
    the library ones, and no multimem kernel variant is selected.  CPU (gloo) ranks are unaffected."""
    if not on_cuda:
        return None
    env = os.environ if env is None else env
    why = []
    if env.get("NCCL_NVLS_ENABLE", "") != "0":
        why.append("NCCL_NVLS_ENABLE=0 is not set in the environment")
    if collectives != "library":
        why.append(f"--collectives {collectives} binds symmetric memory that peers map (use --collectives library)")
    if env.get("ZORSE_RS_ADAM_VARIANT", "0") in ("2", "3"):
        why.append("ZORSE_RS_ADAM_VARIANT selects a multimem kernel")
    if not why:
        return None
    return ("--inject_fault is refused on CUDA devices: a rank that dies while its memory is bound to an NVLink "
            "multicast object faults its peers' GPUs; " + "; ".join(why))


def maybe_inject(fault, rank: int, step: int, keepalive: Optional[Callable[[int], None]] = None,
                 transport=None) -> None:
    """Called between steps, with none of this rank's kernels or collectives in flight.
    `keepalive` (the local watchdog's beat) is called while a stalled rank sleeps, so that the
    stalled rank itself stays silent towards its peers without aborting on its own."""
    if fault is None or fault[0] != rank or fault[1] != step:
        return
    kind = fault[2]
    if kind == "drop" or kind.startswith("delay="):
        if transport is None or not hasattr(transport, "drop_next"):
            raise RuntimeError("message faults need the trainer's p2p_fault_hooks (a FaultyTransport)")
        if kind == "drop":
            transport.drop_next = 1
        else:
            transport.delay_next_s = float(kind[6:])
        return
    if kind == "raise":
        raise RuntimeError(f"injected failure on rank {rank} before step {step}")
    if kind == "exit":
        os._exit(17)
    while True:          # stall: this rank never joins the next step
        time.sleep(1.0)
        if keepalive is not None:
            keepalive(step - 1)
