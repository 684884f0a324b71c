"""Host-side checker for the ordering of pipeline p2p operations.

NCCL matches the messages of a rank pair by order only, and torch runs every p2p operation of
one process group on one internal stream per rank (so they execute strictly in the order the
host issued them); a send finishes only when the matching receive is executing.  Whether a
schedule can deadlock under those rules is a property of the order in which each rank issues
its operations, and can be decided without any GPU:

1. `RecordingTransport` stands in for the real transport while a rank's schedule runs for one
   step in isolation: sends are dropped, receives return zeros, and the sequence of
   (post receive / wait for receive / send) events is recorded.
2. `simulate` replays the recorded programs of all ranks with rendezvous semantics: per rank a
   compute timeline that blocks on receive waits, and per (rank, traffic kind, direction) a FIFO
   of operations; an operation may start once the compute timeline has passed the point where
   it was issued (the transport makes the comm stream wait for the compute stream there) and it
   is at the head of its FIFO; a send/receive pair completes together.

`simulate` returns None when every operation completes, else a description of the stuck heads.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .p2p import Handle


@dataclass
class Event:
    what: str          # "post_recv" | "wait_recv" | "send"
    peer: int
    kind: str          # "act" | "grad"
    tag: int


class RecordingTransport:
    def __init__(self, rank: int, device=None):
        self.rank = rank
        self.device = device or torch.device("cpu")
        self.events: list[Event] = []
        self.bytes_sent = 0

    def send(self, t, dst, tag, kind="act"):
        self.events.append(Event("send", dst, kind, tag))
        return Handle(lambda: None)

    def recv(self, shape, dtype, src, tag, kind="act"):
        self.events.append(Event("post_recv", src, kind, tag))

        def wait():
            self.events.append(Event("wait_recv", src, kind, tag))
            return torch.zeros(shape, dtype=dtype, device=self.device)

        return Handle(wait)

    def flush(self):
        pass


def _queue_key(rank: int, peer: int, kind: str, sending: bool, groups_by_direction: bool):
    if not groups_by_direction:
        return (kind,) if kind is not None else ()
    src, dst = (rank, peer) if sending else (peer, rank)
    return (kind, dst > src)


def simulate(programs: dict[int, list[Event]], *, separate_kinds: bool = True, separate_directions: bool = True,
             serialize_within_group: bool = True) -> Optional[str]:
    """programs: rank -> recorded events of one step. Returns None if everything completes.

    separate_kinds / separate_directions describe how many process groups carry the traffic
    (four when both are True, as `NcclP2P` does; one when both are False).
    serialize_within_group=False models per-pair communicators (ops of different pairs do not
    block one another)."""
    ranks = sorted(programs)
    # per rank: compute timeline = list of event indices; comm ops with their issue index
    queues: dict = {}
    ops = []  # (rank, idx, event)
    for r in ranks:
        for i, e in enumerate(programs[r]):
            if e.what in ("post_recv", "send"):
                sending = e.what == "send"
                key = [r]
                if separate_kinds:
                    key.append(e.kind)
                if separate_directions:
                    src, dst = (r, e.peer) if sending else (e.peer, r)
                    key.append(dst > src)
                if not serialize_within_group:
                    key.append(e.peer)
                queues.setdefault(tuple(key), []).append((r, i, e))
    head = {k: 0 for k in queues}
    pc = {r: 0 for r in ranks}                # compute timeline position (index into programs[r])
    done_recv: set = set()                    # (rank, peer, kind, tag) receives completed

    def advance_compute() -> bool:
        moved = False
        for r in ranks:
            prog = programs[r]
            while pc[r] < len(prog):
                e = prog[pc[r]]
                if e.what == "wait_recv" and (r, e.peer, e.kind, e.tag) not in done_recv:
                    break
                pc[r] += 1
                moved = True
        return moved

    def ready(k):
        if head[k] >= len(queues[k]):
            return None
        r, i, e = queues[k][head[k]]
        return (r, i, e) if pc[r] > i else None   # compute timeline has passed the issue point

    while True:
        progress = advance_compute()
        heads = {k: ready(k) for k in queues}
        for k, h in heads.items():
            if h is None or h[2].what != "send":
                continue
            r, i, e = h
            # find the matching receive at the head of one of the peer's queues
            for k2, h2 in heads.items():
                if h2 is None or h2[2].what != "post_recv":
                    continue
                r2, i2, e2 = h2
                if r2 == e.peer and e2.peer == r and e2.kind == e.kind:
                    if e2.tag != e.tag:
                        return f"order mismatch: rank {r} sends tag {e.tag} to {r2}, which is receiving tag {e2.tag}"
                    head[k] += 1
                    head[k2] += 1
                    done_recv.add((r2, r, e.kind, e.tag))
                    progress = True
                    heads[k] = heads[k2] = None
                    break
        if not progress:
            break
    stuck = []
    for k in queues:
        if head[k] < len(queues[k]):
            r, i, e = queues[k][head[k]]
            stuck.append(f"rank {r}: {e.what} {e.kind} tag {e.tag} peer {e.peer} (compute at {pc[r]}/{len(programs[r])}, issued at {i})")
    for r in ranks:
        if pc[r] < len(programs[r]) and not stuck:
            stuck.append(f"rank {r}: compute stuck at event {pc[r]}")
    return None if not stuck else "deadlock: " + "; ".join(stuck[:8])


def record_programs(cfg, schedule_name: str, model_overrides: Optional[dict] = None,
                    split_parity: Optional[bool] = None, **schedule_kw) -> dict[int, list[Event]]:
    """Runs one step of `schedule_name` for every rank of `cfg` in isolation (CPU, PyTorch ops,
    shard groups of one rank) and returns the recorded p2p programs.  `split_parity`: as `PipelineStage`
    (None: per-boundary groups only for irregular plans, and for schedules asked to post receives ahead)."""
    if split_parity is None and schedule_kw.get("prepost_recv"):
        split_parity = True
    from ..engine.zero import EngineConfig, Streams
    from ..ops.api import get_ops
    from .groups import Group, StageGroups
    from .p2p_plan import create_static_comm_plans
    from .schedules import build_schedule
    from .stage import PipelineStage

    plans = create_static_comm_plans(cfg)
    dev = torch.device("cpu")
    ops = get_ops("ref")
    out = {}
    g = torch.Generator().manual_seed(0)
    M, B, S = cfg.num_microbatches, cfg.microbatch_size, cfg.sequence_length
    inputs = {i: torch.randint(0, cfg.vocab_size, (B, S), generator=g) for i in range(M)}
    from .p2p import LocalMailbox

    for r in sorted(plans):
        tp = RecordingTransport(r)
        box = LocalMailbox()
        ecfg = EngineConfig(compute_dtype=torch.float32, reduce_dtype=torch.float32)
        streams = Streams(dev)
        stages = [PipelineStage(cfg, st, rank=r, device=dev, ops=ops, engine_cfg=ecfg,
                                groups=StageGroups(Group((r,)), Group((r,))), streams=streams,
                                pattern=plans[r].stages[st.stage_id], transport=tp, model_overrides=model_overrides,
                                local_mailbox=box, split_parity=split_parity)
                  for st in cfg.stages_of_rank(r)]
        sched = build_schedule(schedule_name, stages, cfg, **schedule_kw)
        sched.step(0, inputs, inputs)
        out[r] = tp.events
    return out


def preflight(cfg, schedule_name: str, **schedule_kw) -> Optional[str]:
    """Replays the p2p program that `schedule_name` issues for `cfg` (same stages, ranks, microbatch counts and
    schedule code, on a few-parameter stand-in model on the CPU) under the rules above.  Returns None when every
    transfer completes, else a description of the wait cycle: a job whose program cannot complete must not be
    started on GPUs, where it would sit in NCCL kernels until somebody's timeout.  Takes seconds."""
    import dataclasses

    from ..models import registry

    if len(cfg.stages) < 2:
        return None
    if registry.get_spec(cfg.model_name).family == "vit":
        return None        # image inputs: the stand-in below feeds token ids
    small = dataclasses.replace(cfg, sequence_length=8, vocab_size=64, tensor_parallel_size=1)
    tiny = {"hidden": 16, "heads": 2, "kv_heads": 2, "ffn": 32, "max_positions": 0} \
        if registry.get_spec(cfg.model_name).max_positions == 0 else {"hidden": 16, "heads": 2, "kv_heads": 2, "ffn": 32}
    threads = torch.get_num_threads()
    torch.set_num_threads(1)          # tiny tensors, and every rank of a node runs this at the same time
    try:
        progs = record_programs(small, schedule_name, model_overrides=tiny, **schedule_kw)
    finally:
        torch.set_num_threads(threads)
    return simulate(progs)
