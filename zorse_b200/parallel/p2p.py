"""Point-to-point transports for activations and activation gradients between stages.

`NcclP2P`  – NCCL send/recv issued on two side streams with event hand-off to the compute
             stream (the reference does the same with two class-wide streams,
             zorse_utils/pipeline_comm.py:322-402).  NCCL matches messages of a rank pair by
             order only, and torch serialises all p2p operations of one pair and one process
             group on one internal stream; a send queued behind an unmatched send of the
             other direction is the classic pipeline deadlock the reference works around with
             its "sync" schedules and its Gloo path.  Here the four kinds of traffic
             (activations / gradients x towards higher / lower rank) each get their own
             process group, so every queue carries one kind in one direction, in increasing
             (or, for gradients, decreasing) microbatch order on both ends.
`GlooP2P`  – tagged Gloo send/recv; CUDA tensors are staged through pinned host buffers on a
             copy stream (reference zorse_utils/gloo_pipeline_comm.py:8-160).  Also the CPU path.
`LoopbackP2P` – in-process mailbox for single-process tests.
"""
from __future__ import annotations

import datetime

import torch
import torch.distributed as dist

from ..utils import stream_check as SC


class Handle:
    """Result of an asynchronous transfer. wait() returns the received tensor (None for sends)."""

    def __init__(self, wait_fn):
        self._wait_fn = wait_fn
        self._done = False
        self._val = None

    def wait(self):
        if not self._done:
            self._val = self._wait_fn()
            self._done = True
        return self._val


class NcclP2P:
    def __init__(self, device: torch.device, timeout_s: float = 300.0, streams=None, split_parity: bool = False):
        # kinds of traffic, each with an "up" and a "down" group; with split_parity the boundaries of even
        # and odd index get their own groups (needed for irregular routing, see PipelineStage)
        self.KINDS = ("act0", "act1", "grad0", "grad1") if split_parity else ("act", "grad")
        self.device = device
        self.streams = streams  # engine Streams: brackets receive waits for exposed-communication accounting
        self.rank = dist.get_rank()
        self.send_stream = torch.cuda.Stream(device=device)
        self.recv_stream = torch.cuda.Stream(device=device)
        to = datetime.timedelta(seconds=timeout_s)
        # collective: every rank creates the same four world-wide groups in the same order
        self.groups = {(k, up): dist.new_group(backend="nccl", timeout=to) for k in self.KINDS for up in (True, False)}
        self._pending: list = []
        self.bytes_sent = 0

    def _group(self, kind: str, src: int, dst: int):
        return self.groups[(kind, dst > src)]

    @staticmethod
    def _post(op, tensor, peer: int, group):
        """One send or receive as a batch of one: the batched form runs inside an NCCL group call on the
        process group's communicator, which is what torch wants for p2p on an eagerly initialised group
        (the unbatched form is treated as a collective of the whole group there, with a warning per call).
        Ordering is unchanged: one queue per process group and device either way."""
        return dist.batch_isend_irecv([dist.P2POp(op, tensor, peer, group=group)])[-1]

    def send(self, t: torch.Tensor, dst: int, tag: int, kind: str = "act") -> Handle:
        cur = torch.cuda.current_stream()
        SC.wrote(("p2p_src", id(t)), cur)
        self.send_stream.wait_stream(cur)
        with torch.cuda.stream(self.send_stream):
            SC.read(("p2p_src", id(t)), label="NCCL send of a tensor the compute stream produced")
            work = self._post(dist.isend, t, dst, self._group(kind, self.rank, dst))
        t.record_stream(self.send_stream)
        self.bytes_sent += t.numel() * t.element_size()
        self._pending.append((work, t))
        return Handle(lambda: work.wait())

    def recv(self, shape, dtype, src: int, tag: int, kind: str = "act") -> Handle:
        cur = torch.cuda.current_stream()
        buf = torch.empty(shape, dtype=dtype, device=self.device)
        self.recv_stream.wait_stream(cur)
        with torch.cuda.stream(self.recv_stream):
            work = self._post(dist.irecv, buf, src, self._group(kind, src, self.rank))
        buf.record_stream(self.recv_stream)

        def wait():
            with torch.cuda.stream(self.recv_stream):
                work.wait()
                SC.wrote(("p2p_dst", id(buf)))
            if self.streams is not None:
                self.streams.wait_stream(self.recv_stream, kind="pipeline")
            else:
                torch.cuda.current_stream().wait_stream(self.recv_stream)
            SC.read(("p2p_dst", id(buf)), label="compute on a received tensor")
            return buf

        return Handle(wait)

    def flush(self) -> None:
        """Waits (stream-wise) for every send issued so far."""
        if not self._pending:
            return
        with torch.cuda.stream(self.send_stream):
            for work, _ in self._pending:
                work.wait()
        self._pending.clear()
        torch.cuda.current_stream().wait_stream(self.send_stream)


class P2PTimeout(RuntimeError):
    """A pipeline message did not arrive in time; the text names the message."""


class GlooP2P:
    def __init__(self, device: torch.device, group=None, recv_timeout_s: float | None = None):
        """`recv_timeout_s`: how long a receive may wait for its message before `P2PTimeout` is raised with the
        sender, tag and kind of the missing message (None: the process group's own timeout applies)."""
        self.device = device
        self.group = group
        self.recv_timeout_s = recv_timeout_s
        self.cuda = device.type == "cuda"
        if self.cuda:
            self.copy_send = torch.cuda.Stream(device=device)
            self.copy_recv = torch.cuda.Stream(device=device)
        self._pending: list = []
        self.bytes_sent = 0

    def send(self, t: torch.Tensor, dst: int, tag: int, kind: str = "act") -> Handle:
        if self.cuda:
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            self.copy_send.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.copy_send):
                host.copy_(t, non_blocking=True)
            t.record_stream(self.copy_send)
            self.copy_send.synchronize()
        else:
            host = t.contiguous()
        work = dist.isend(host, dst, group=self.group, tag=tag)
        self.bytes_sent += t.numel() * t.element_size()
        h = Handle(lambda: work.wait())
        self._pending.append((h, host))
        return h

    def recv(self, shape, dtype, src: int, tag: int, kind: str = "act") -> Handle:
        host = torch.empty(shape, dtype=dtype, device="cpu", pin_memory=self.cuda)
        work = dist.irecv(host, src, group=self.group, tag=tag)

        def wait():
            if self.recv_timeout_s is None:
                work.wait()
            else:
                try:
                    done = work.wait(datetime.timedelta(seconds=self.recv_timeout_s))
                except RuntimeError as e:
                    raise P2PTimeout(f"no {kind} message with tag {tag} from rank {src} within {self.recv_timeout_s:g}s "
                                     f"({str(e).splitlines()[0][:120]})") from e
                if done is False:
                    raise P2PTimeout(f"no {kind} message with tag {tag} from rank {src} within {self.recv_timeout_s:g}s")
            if not self.cuda:
                return host
            with torch.cuda.stream(self.copy_recv):
                dev = host.to(self.device, non_blocking=True)
            torch.cuda.current_stream().wait_stream(self.copy_recv)
            dev.record_stream(torch.cuda.current_stream())
            return dev

        return Handle(wait)

    def flush(self) -> None:
        for h, _ in self._pending:
            h.wait()  # idempotent: a Gloo work object must not be waited on twice
        self._pending.clear()


class LocalMailbox:
    """Hand-off between two stages of the same rank (a plan may put consecutive stages on one rank
    group, so a microbatch's next owner can be the rank itself).  Neither NCCL nor Gloo sends to the
    calling rank; the tensor simply stays where it is: producer and consumer both run on the rank's
    compute stream, in program order."""

    def __init__(self):
        self.box: dict = {}

    def send(self, t, tag: int) -> Handle:
        self.box[tag] = t
        return Handle(lambda: None)

    def recv(self, tag: int) -> Handle:
        def wait():
            if tag not in self.box:
                raise RuntimeError(f"local hand-off {tag} is received before it was sent (schedule order)")
            return self.box.pop(tag)

        return Handle(wait)


class LoopbackP2P:
    """Mailbox shared by simulated ranks of one process: {(src, dst, tag): tensor}."""

    def __init__(self, rank: int, mailbox: dict):
        self.rank, self.mailbox = rank, mailbox
        self.bytes_sent = 0

    def send(self, t, dst, tag, kind="act"):
        self.mailbox[(self.rank, dst, tag)] = t.detach().clone()
        self.bytes_sent += t.numel() * t.element_size()
        return Handle(lambda: None)

    def recv(self, shape, dtype, src, tag, kind="act"):
        def wait():
            return self.mailbox.pop((src, self.rank, tag))

        return Handle(wait)

    def flush(self):
        pass


class FaultyTransport:
    """Host-side fault injection on the pipeline's messages (failure-detection tests; nothing on a device is made
    to fault): the next `drop_next` sends are silently dropped, the next send is delayed by `delay_next_s` seconds."""

    def __init__(self, inner):
        self.inner = inner
        self.drop_next = 0
        self.delay_next_s = 0.0
        self.dropped: list = []

    def send(self, t, dst, tag, kind="act"):
        if self.drop_next > 0:
            self.drop_next -= 1
            self.dropped.append((dst, tag, kind))
            return Handle(lambda: None)
        if self.delay_next_s > 0:
            import time

            d, self.delay_next_s = self.delay_next_s, 0.0
            time.sleep(d)
        return self.inner.send(t, dst, tag, kind)

    def recv(self, shape, dtype, src, tag, kind="act"):
        return self.inner.recv(shape, dtype, src, tag, kind)

    def flush(self):
        self.inner.flush()

    @property
    def bytes_sent(self):
        return self.inner.bytes_sent


class LaneTransport:
    """With tensor parallelism the plan numbers lanes, and slice t of lane a talks to slice t of lane b:
    this wrapper turns lane numbers into process ranks (lane * tp + t) for the transport under it."""

    def __init__(self, inner, tp: int, index: int):
        self.inner, self.tp, self.index = inner, tp, index

    def send(self, t, dst, tag, kind="act"):
        return self.inner.send(t, dst * self.tp + self.index, tag, kind)

    def recv(self, shape, dtype, src, tag, kind="act"):
        return self.inner.recv(shape, dtype, src * self.tp + self.index, tag, kind)

    def flush(self):
        self.inner.flush()

    @property
    def bytes_sent(self):
        return self.inner.bytes_sent


def make_transport(device: torch.device, use_gloo: bool = False, gloo_group=None, streams=None,
                   split_parity: bool = False, recv_timeout_s: float | None = None):
    if not (dist.is_available() and dist.is_initialized()):
        return LoopbackP2P(0, {})
    if device.type == "cuda" and not use_gloo:
        return NcclP2P(device, streams=streams, split_parity=split_parity)
    return GlooP2P(device, gloo_group, recv_timeout_s=recv_timeout_s)
