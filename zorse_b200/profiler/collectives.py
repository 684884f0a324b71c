"""Collective benchmarks: the patterns the planner needs to cost ZeRO traffic.

Classes with `.execute()` as in the reference's research tool (utils/comm_patterns.py:1-403):
all-reduce, all-gather, reduce-scatter, broadcast; all-gather / reduce-scatter restricted to the
ranks of one node or to the ranks of equal local index across nodes (`node_groups`); hybrid
reduce-scatter (reduce-scatter inside a group + all-reduce across groups); 2-hop reduce-scatter
and "ZeRO 2.5" (the same with an all-gather back across the outer group); its world-wide
list-based form; uneven (list based) all-gather / reduce-scatter by ratios or by sizes — timed
with CUDA events (max over ranks) instead of profiler traces.  `fit_switch_model` turns timings at several sizes into the alpha / bandwidth pair
of `planner/comm_model.switch_collective_ms`.
"""
from __future__ import annotations

import statistics
import time
from typing import Sequence

import torch
import torch.distributed as dist


class Pattern:
    name = "pattern"

    def __init__(self, numel: int, dtype=torch.bfloat16, group=None, device=None):
        self.group = group
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self.R = dist.get_world_size(group)
        self.numel = (numel + self.R - 1) // self.R * self.R
        self.dtype = dtype
        self.full = torch.ones(self.numel, dtype=dtype, device=self.device)
        self.shard = torch.ones(self.numel // self.R, dtype=dtype, device=self.device)

    def bytes(self) -> int:
        return self.numel * self.full.element_size()

    def execute(self):
        raise NotImplementedError


class AllReduce(Pattern):
    name = "all_reduce"

    def execute(self):
        dist.all_reduce(self.full, group=self.group)


class AllGather(Pattern):
    name = "all_gather"

    def execute(self):
        dist.all_gather_into_tensor(self.full, self.shard, group=self.group)


class ReduceScatter(Pattern):
    name = "reduce_scatter"

    def execute(self):
        dist.reduce_scatter_tensor(self.shard, self.full, group=self.group)


class Broadcast(Pattern):
    name = "broadcast"

    def execute(self):
        dist.broadcast(self.full, src=dist.get_global_rank(self.group, 0) if self.group else 0, group=self.group)


class HybridReduceScatter(Pattern):
    """Reduce-scatter inside the shard group, then all-reduce of the shard across replicate groups."""
    name = "hybrid_reduce_scatter"

    def __init__(self, numel, dtype=torch.bfloat16, shard_group=None, replicate_group=None, device=None):
        super().__init__(numel, dtype, shard_group, device)
        self.replicate_group = replicate_group

    def execute(self):
        dist.reduce_scatter_tensor(self.shard, self.full, group=self.group)
        if self.replicate_group is not None:
            dist.all_reduce(self.shard, group=self.replicate_group)


def node_groups(local_size: int | None = None):
    """(intra-node group of this rank, inter-node group of this rank): the ranks of this rank's node, and the ranks
    with this rank's local index on every node (reference utils/comm.py:124-160).  Collective: every rank creates
    every group, in the same order.  `local_size` defaults to LOCAL_WORLD_SIZE, else the whole job is one node."""
    import os

    world, me = dist.get_world_size(), dist.get_rank()
    local = int(local_size or os.environ.get("LOCAL_WORLD_SIZE", world))
    if world % local:
        raise ValueError(f"{world} ranks do not split into nodes of {local}")
    intra = inter = None
    for node in range(world // local):
        g = dist.new_group(list(range(node * local, (node + 1) * local)))
        if me // local == node:
            intra = g
    for idx in range(local):
        g = dist.new_group(list(range(idx, world, local)))
        if me % local == idx:
            inter = g
    return intra, inter


class ScopedAllGather(Pattern):
    """All-gather of a world-wide message's pieces inside one scope: with the intra-node group every rank
    contributes 1 / world of the message and ends up with its node's part; with the inter-node group 1 / world
    again, gathered across the nodes (reference IntraNodeAllGather / InterNodeAllGather)."""
    name = "scoped_all_gather"

    def __init__(self, numel, dtype=torch.bfloat16, scope_group=None, device=None, name=None):
        super().__init__(numel, dtype, scope_group, device)
        world = dist.get_world_size()
        piece = max(self.numel // world, 1)
        self.shard = torch.ones(piece, dtype=dtype, device=self.device)
        self.full = torch.ones(piece * self.R, dtype=dtype, device=self.device)
        if name:
            self.name = name

    def bytes(self) -> int:
        return self.full.numel() * self.full.element_size()

    def execute(self):
        dist.all_gather_into_tensor(self.full, self.shard, group=self.group)


class ScopedReduceScatter(ScopedAllGather):
    name = "scoped_reduce_scatter"

    def execute(self):
        dist.reduce_scatter_tensor(self.shard, self.full, group=self.group)


def IntraNodeAllGather(numel, dtype=torch.bfloat16, device=None, groups=None):
    return ScopedAllGather(numel, dtype, (groups or node_groups())[0], device, "intra_node_all_gather")


def InterNodeAllGather(numel, dtype=torch.bfloat16, device=None, groups=None):
    return ScopedAllGather(numel, dtype, (groups or node_groups())[1], device, "inter_node_all_gather")


def IntraNodeReduceScatter(numel, dtype=torch.bfloat16, device=None, groups=None):
    return ScopedReduceScatter(numel, dtype, (groups or node_groups())[0], device, "intra_node_reduce_scatter")


def InterNodeReduceScatter(numel, dtype=torch.bfloat16, device=None, groups=None):
    return ScopedReduceScatter(numel, dtype, (groups or node_groups())[1], device, "inter_node_reduce_scatter")


class ReduceScatter2Hop(Pattern):
    """Reduce-scatter inside the inner group, then reduce-scatter of the result across the outer group; with
    `gather_back` the outer shards are all-gathered again, so that every rank of the inner group ends with its
    fully reduced inner shard (the reference's `Zero_2_5`; without it, its `ReduceScatter2Hop`)."""
    name = "reduce_scatter_2hop"
    gather_back = False

    def __init__(self, numel, dtype=torch.bfloat16, inner_group=None, outer_group=None, device=None):
        super().__init__(numel, dtype, inner_group, device)
        self.outer = outer_group
        self.Ro = dist.get_world_size(outer_group) if outer_group is not None else 1
        n2 = self.shard.numel() // self.Ro * self.Ro
        self.shard2 = torch.ones(max(n2 // self.Ro, 1), dtype=dtype, device=self.device)
        self.n2 = n2

    def execute(self):
        dist.reduce_scatter_tensor(self.shard, self.full, group=self.group)
        if self.outer is not None and self.Ro > 1:
            dist.reduce_scatter_tensor(self.shard2, self.shard[: self.n2], group=self.outer)
            if self.gather_back:
                dist.all_gather_into_tensor(self.shard[: self.n2], self.shard2, group=self.outer)


class Zero25(ReduceScatter2Hop):
    name = "zero_2_5"
    gather_back = True


class Zero25Global(Pattern):
    """The same result over one flat group: list-based reduce-scatter of the whole message over every rank, then
    an all-gather of the reduced pieces (reference `Zero_2_5_Global`)."""
    name = "zero_2_5_global"

    def __init__(self, numel, dtype=torch.bfloat16, group=None, device=None):
        super().__init__(numel, dtype, group, device)
        self.pieces = list(self.full.split(self.numel // self.R))

    def execute(self):
        dist.reduce_scatter(self.shard, self.pieces, group=self.group)
        dist.all_gather_into_tensor(self.full, self.shard, group=self.group)


class UnevenAllGather(Pattern):
    """List-based all-gather with per-rank shard sizes given by `ratios`."""
    name = "uneven_all_gather"

    def __init__(self, numel, ratios: Sequence[float] | None = None, dtype=torch.bfloat16, group=None, device=None,
                 sizes: Sequence[int] | None = None):
        """Per-rank piece sizes: `sizes` (elements) when given, else `numel` split by `ratios`."""
        super().__init__(numel, dtype, group, device)
        if sizes is None:
            tot = sum(ratios)
            sizes = [max(int(self.numel * r / tot), 1) for r in ratios]
        if len(sizes) != self.R:
            raise ValueError(f"{len(sizes)} piece sizes for a group of {self.R}")
        self.parts = [torch.ones(s, dtype=dtype, device=self.device) for s in sizes]
        self.mine = self.parts[dist.get_rank(group)].clone()

    def _owner(self, q: int) -> int:
        return dist.get_global_rank(self.group, q) if self.group is not None else q

    def execute(self):
        if self.device.type == "cuda":
            dist.all_gather(self.parts, self.mine, group=self.group)
            return
        # Gloo has no list form with unequal sizes: one broadcast per piece (what the ZeRO engine does for
        # unequal shards on CPU ranks)
        self.parts[dist.get_rank(self.group)].copy_(self.mine)
        for q, part in enumerate(self.parts):
            dist.broadcast(part, src=self._owner(q), group=self.group)


class UnevenReduceScatter(UnevenAllGather):
    name = "uneven_reduce_scatter"

    def execute(self):
        if self.device.type == "cuda":
            dist.reduce_scatter(self.mine, self.parts, group=self.group)
            return
        me = dist.get_rank(self.group)
        for q, part in enumerate(self.parts):
            buf = part.clone()
            dist.reduce(buf, dst=self._owner(q), group=self.group)
            if q == me:
                self.mine.copy_(buf)


def time_pattern(p: Pattern, warmup: int = 3, trials: int = 10) -> dict:
    """avg / min / max / std in ms (max over ranks per trial) and algorithmic bandwidth in MB/s."""
    cuda = p.device.type == "cuda"
    for _ in range(warmup):
        p.execute()
    ts = []
    for _ in range(trials):
        if cuda:
            torch.cuda.synchronize()
        dist.barrier(group=p.group)
        if cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            p.execute()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], device=p.device)
        else:
            t0 = time.perf_counter()
            p.execute()
            t = torch.tensor([(time.perf_counter() - t0) * 1e3])
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=p.group)
        ts.append(float(t.item()))
    avg = sum(ts) / len(ts)
    return {"avg_time_ms": avg, "min_time_ms": min(ts), "max_time_ms": max(ts),
            "std_time_ms": statistics.pstdev(ts), "bandwidth_mbps": p.bytes() / 1e6 / (avg / 1e3),
            "tensor_size_mb": p.bytes() / 2**20, "num_parameters": p.numel, "world_size": p.R}


def fit_switch_model(sizes_bytes: Sequence[float], times_ms: Sequence[float], R: int) -> dict:
    """Least squares of t = alpha + (R-1)/R * bytes / BW  ->  {'alpha_ms', 'bandwidth_gbs'}."""
    xs = [(R - 1) / R * s / 1e9 for s in sizes_bytes]  # GB on the wire per rank
    n = len(xs)
    mx, my = sum(xs) / n, sum(times_ms) / n
    den = sum((x - mx) ** 2 for x in xs) or 1e-30
    slope = sum((x - mx) * (y - my) for x, y in zip(xs, times_ms)) / den  # ms per GB
    alpha = max(my - slope * mx, 0.0)
    return {"alpha_ms": alpha, "bandwidth_gbs": 1e3 / slope if slope > 0 else float("inf")}
