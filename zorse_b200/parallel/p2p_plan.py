"""Static routing of microbatches between pipeline stages.

Stages may have different widths and every rank of a stage may run a different number of
microbatches (heterogeneous data parallelism), so "who sends microbatch g to whom" is a
many-to-many plan fixed before training, as in the reference
(zorse_utils/pipeline_comm.py:17-312).  Here the plan is built from one rule: every stage
orders the M global microbatches 0..M-1 and hands them to its ranks by a largest-remainder
interleave of `num_microbatches_per_rank` (which reduces to `g % n` for an even split, the
reference's even plan at :99-171); microbatch g then travels from its owner on stage s to
its owner on stage s+1.  Ranks work through their microbatches in increasing g, so every
pair of ranks sees its messages in one consistent order.

Tags are unique per (stage boundary, microbatch, direction): `2*(b*M + g)` forward,
`2*(b*M + g) + 1` backward.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence


def interleave_owners(counts: Sequence[int]) -> list[int]:
    """Owner (index into the stage's rank list) of each of sum(counts) microbatches, spreading
    every rank's share evenly over the sequence. counts=[2,2] -> [0,1,0,1]; [3,1] -> [0,0,1,0]."""
    total = sum(counts)
    done = [0] * len(counts)
    out = []
    for g in range(total):
        # the rank that is furthest behind its ideal share (g+1) * counts[k] / total
        best, best_def = -1, None
        for k, c in enumerate(counts):
            if done[k] >= c:
                continue
            deficit = (g + 1) * c / total - done[k]
            if best_def is None or deficit > best_def + 1e-12:
                best, best_def = k, deficit
        done[best] += 1
        out.append(best)
    return out


@dataclass
class StageCommPattern:
    """For one local stage of one rank: its microbatches (global ids, increasing) and, per
    local microbatch index, the peer rank + tag for each of the four transfers (None = no transfer)."""
    stage_id: int
    microbatches: list[int] = field(default_factory=list)
    fwd_recv: list = field(default_factory=list)   # (src_rank, tag) | None
    fwd_send: list = field(default_factory=list)   # (dst_rank, tag) | None
    bwd_recv: list = field(default_factory=list)   # (src_rank, tag) | None  (gradient from next stage)
    bwd_send: list = field(default_factory=list)   # (dst_rank, tag) | None  (gradient to previous stage)


@dataclass
class RankCommPlan:
    rank: int
    stages: dict[int, StageCommPattern] = field(default_factory=dict)


def latency_owners(counts: Sequence[int], latency: Sequence[float], receiver: bool) -> list[int]:
    """Owner (index into the stage's rank list) of each microbatch when the ranks differ in speed
    (reference zorse_utils/pipeline_comm.py:193-303, a greedy matching per stage boundary).

    A rank with `latency` ms per microbatch finishes its i-th microbatch at `latency * i`.  On the sending
    side of a boundary the g-th microbatch is the g-th to finish (`receiver=False`: sorted by completion
    time, slower rank first on ties, as the reference's tuples sort); on the receiving side it goes to the rank with the g-th largest amount
    of work still ahead of it, `latency * (count - i)` (`receiver=True`), so the ranks that need longest are
    fed first.  Equal ranks with equal counts get the plain round-robin either way."""
    items = []
    for k, (c, lat) in enumerate(zip(counts, latency)):
        for i in range(c):
            items.append(((-lat * (c - i), -lat, -k) if receiver else (lat * i, -lat, k)))
    items.sort()
    return [abs(k) for _, _, k in items]


def stage_owners(stage, cfg=None, position: int = 0) -> list[int]:
    """Global rank owning each global microbatch on `stage`.  With `cfg.comm_plan == "latency"` and per-rank
    latencies in `cfg.rank_latency_ms`, the first stage deals its microbatches in the order they finish and every
    later stage takes them in the order of the work its ranks still have ahead (see `latency_owners`)."""
    lat = getattr(cfg, "rank_latency_ms", None) if cfg is not None else None
    if cfg is not None and getattr(cfg, "comm_plan", "interleave") == "latency" and lat \
            and all(r in lat for r in stage.gpu_ranks):
        idx = latency_owners(stage.num_microbatches_per_rank, [lat[r] * stage.num_layers for r in stage.gpu_ranks],
                             receiver=position > 0)
    else:
        idx = interleave_owners(stage.num_microbatches_per_rank)
    return [stage.gpu_ranks[k] for k in idx]


def create_static_comm_plans(cfg) -> dict[int, RankCommPlan]:
    """rank -> plan, for every rank named in the config."""
    stages = cfg.stages
    M = cfg.num_microbatches
    owners = [stage_owners(s, cfg, i) for i, s in enumerate(stages)]
    plans: dict[int, RankCommPlan] = {}
    for si, st in enumerate(stages):
        for r in st.gpu_ranks:
            plans.setdefault(r, RankCommPlan(r)).stages[st.stage_id] = StageCommPattern(st.stage_id)
    for si, st in enumerate(stages):
        for g in range(M):
            r = owners[si][g]
            pat = plans[r].stages[st.stage_id]
            pat.microbatches.append(g)
            if si > 0:
                tag = 2 * ((si - 1) * M + g)
                pat.fwd_recv.append((owners[si - 1][g], tag))
                pat.bwd_send.append((owners[si - 1][g], tag + 1))
            else:
                pat.fwd_recv.append(None)
                pat.bwd_send.append(None)
            if si + 1 < len(stages):
                tag = 2 * (si * M + g)
                pat.fwd_send.append((owners[si + 1][g], tag))
                pat.bwd_recv.append((owners[si + 1][g], tag + 1))
            else:
                pat.fwd_send.append(None)
                pat.bwd_recv.append(None)
    validate_static_comm_plans(cfg, plans)
    return plans


def validate_static_comm_plans(cfg, plans: dict[int, RankCommPlan]) -> None:
    """Every microbatch crosses every boundary exactly once each way, send and receive sides
    mirror each other, tags are unique, and every rank runs the count the config gives it."""
    M = cfg.num_microbatches
    sends, recvs = {}, {}
    for r, plan in plans.items():
        for sid, pat in plan.stages.items():
            st = cfg.stages[sid]
            want = st.num_microbatches_per_rank[st.gpu_ranks.index(r)]
            if len(pat.microbatches) != want:
                raise AssertionError(f"rank {r} stage {sid}: {len(pat.microbatches)} microbatches, config says {want}")
            if pat.microbatches != sorted(pat.microbatches):
                raise AssertionError(f"rank {r} stage {sid}: microbatches not in increasing order")
            for g, fs, fr, bs, br in zip(pat.microbatches, pat.fwd_send, pat.fwd_recv, pat.bwd_send, pat.bwd_recv):
                for kind, ent in (("send", fs), ("send", bs)):
                    if ent is not None:
                        key = (r, ent[0], ent[1])
                        if key in sends:
                            raise AssertionError(f"duplicate send {key}")
                        sends[key] = g
                for ent in (fr, br):
                    if ent is not None:
                        key = (ent[0], r, ent[1])
                        if key in recvs:
                            raise AssertionError(f"duplicate recv {key}")
                        recvs[key] = g
    if sends.keys() != recvs.keys():
        raise AssertionError(f"unmatched transfers: {set(sends) ^ set(recvs)}")
    for key in sends:
        if sends[key] != recvs[key]:
            raise AssertionError(f"transfer {key} carries different microbatches on its two ends")
    tags = [k[2] for k in sends]
    if len(tags) != len(set(tags)):
        raise AssertionError("tags are not unique")
    expect = 2 * M * (len(cfg.stages) - 1)
    if len(sends) != expect:
        raise AssertionError(f"{len(sends)} transfers planned, expected {expect}")


def is_regular(cfg) -> bool:
    """True when every stage has the same width and every rank the same number of microbatches:
    microbatch g then sits on rank `g % width` of every stage and all ranks of a column see the
    same sequence of microbatches (the case the classic 1F1B order and one-ahead receives assume)."""
    widths = {len(s.gpu_ranks) for s in cfg.stages}
    counts = {c for s in cfg.stages for c in s.num_microbatches_per_rank}
    return len(widths) == 1 and len(counts) == 1


def plan_1f1b_order(cfg, f_cost: float = 1.0, b_cost: float = 2.0) -> dict[int, list[tuple[str, int]]]:
    """Per rank, the order of forward ("F") and backward ("B") passes over its local microbatches
    for a one-forward-one-backward schedule on ANY static routing (mixed stage widths, uneven
    microbatch counts).

    With many-to-many routing the ranks of a stage see different subsequences of the global
    microbatch order, and the classic rule (P - s - 1 warm-up forwards, then strict alternation)
    can make a rank wait for a gradient whose forward depends on an activation that same rank
    would only produce later.  The order is therefore taken from a list-scheduling run of the
    whole pipeline with unit costs (forward 1, backward 2 per layer): at every step the pass
    that can start earliest is placed, backward before forward on ties, at most `P - s` forwards
    in flight per rank (raised only if nothing could be placed).  Every rank computes the same
    plan from the config alone; issuing passes in this order cannot deadlock because the run
    itself is one valid execution.  Ranks host one stage each."""
    stages = cfg.stages
    P, M = len(stages), cfg.num_microbatches
    owners = [stage_owners(s, cfg, i) for i, s in enumerate(stages)]
    stage_of: dict[int, int] = {}
    for si, s in enumerate(stages):
        for r in s.gpu_ranks:
            if r in stage_of:
                raise ValueError("plan_1f1b_order: a rank hosts several stages")
            stage_of[r] = si
    local = {r: [g for g in range(M) if owners[si][g] == r] for r, si in stage_of.items()}
    nf = {r: 0 for r in stage_of}
    nb = {r: 0 for r in stage_of}
    free = {r: 0.0 for r in stage_of}
    order: dict[int, list] = {r: [] for r in stage_of}
    act_ready = [[0.0 if si == 0 else None for _ in range(M)] for si in range(P)]
    grad_ready = [[None] * M for _ in range(P)]
    extra = 0
    remaining = sum(len(v) for v in local.values())
    while remaining:
        best = None
        for r in sorted(stage_of):
            si = stage_of[r]
            if nb[r] < nf[r]:
                ready = grad_ready[si][local[r][nb[r]]]
                if ready is not None:
                    cand = (max(free[r], ready), 0, r, "B")
                    best = cand if best is None or cand < best else best
            if nf[r] < len(local[r]) and nf[r] - nb[r] < P - si + extra:
                ready = act_ready[si][local[r][nf[r]]]
                if ready is not None:
                    cand = (max(free[r], ready), 1, r, "F")
                    best = cand if best is None or cand < best else best
        if best is None:
            extra += 1          # every rank is at its in-flight limit: allow one more forward
            if extra > M:
                raise RuntimeError("plan_1f1b_order: no pass can be placed (inconsistent routing)")
            continue
        start, _, r, op = best
        si = stage_of[r]
        n_layers = stages[si].num_layers
        if op == "F":
            g = local[r][nf[r]]
            end = start + f_cost * n_layers
            if si + 1 < P:
                act_ready[si + 1][g] = end
            else:
                grad_ready[si][g] = end       # the last stage can turn around at once
            order[r].append(("F", nf[r]))
            nf[r] += 1
        else:
            g = local[r][nb[r]]
            end = start + b_cost * n_layers
            if si > 0:
                grad_ready[si - 1][g] = end
            order[r].append(("B", nb[r]))
            nb[r] += 1
            remaining -= 1
        free[r] = end
    return order
