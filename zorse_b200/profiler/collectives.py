"""Collective benchmarks: the patterns the planner needs to cost ZeRO traffic.

Classes with `.execute()` as in the reference's research tool (utils/comm_patterns.py:1-403):
all-reduce, all-gather, reduce-scatter, hybrid reduce-scatter (reduce-scatter inside a group
+ all-reduce across groups), 2-hop reduce-scatter, uneven (list based) all-gather /
reduce-scatter, broadcast — timed with CUDA events (max over ranks) instead of profiler
traces.  `fit_switch_model` turns timings at several sizes into the alpha / bandwidth pair
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


class ReduceScatter2Hop(Pattern):
    """Reduce-scatter inside the inner group, reduce-scatter of the result across the outer
    group, all-gather back across the outer group (the reference's "ZeRO 2.5" pattern)."""
    name = "reduce_scatter_2hop"

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
            dist.all_gather_into_tensor(self.shard[: self.n2], self.shard2, group=self.outer)


class UnevenAllGather(Pattern):
    """List-based all-gather with per-rank shard sizes given by `ratios`."""
    name = "uneven_all_gather"

    def __init__(self, numel, ratios: Sequence[float], dtype=torch.bfloat16, group=None, device=None):
        super().__init__(numel, dtype, group, device)
        tot = sum(ratios)
        sizes = [max(int(self.numel * r / tot), 1) for r in ratios]
        self.parts = [torch.ones(s, dtype=dtype, device=self.device) for s in sizes]
        self.mine = self.parts[dist.get_rank(group)].clone()

    def execute(self):
        dist.all_gather(self.parts, self.mine, group=self.group)


class UnevenReduceScatter(UnevenAllGather):
    name = "uneven_reduce_scatter"

    def execute(self):
        dist.reduce_scatter(self.mine, self.parts, group=self.group)


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
