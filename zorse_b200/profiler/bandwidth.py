"""Point-to-point bandwidth probe between ranks (torchrun worker logic).

`measure_pair`: `parallel` concurrent isend/irecv of `numel` float32 between two ranks, warm-up
then timed trials; NCCL on GPUs (CUDA events), Gloo on CPU tensors (wall clock) — the
reference's probe (benchmark_gpu_bandwidth.py:26-93) with one difference in units: results are
GB/s and seconds per message, named as such.  `measure_all_pairs_concurrent` drives every
GPU's links at once, which is what a collective sees on an NVSwitch domain.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


def measure_pair(src: int, dst: int, numel: int = 10_000_000, parallel: int = 1, warmup: int = 5, trials: int = 10,
                 device=None, group=None) -> dict:
    """Called by every rank; returns {'bandwidth_gbs', 'latency_s'} (valid on src and dst)."""
    rank = dist.get_rank()
    device = device or torch.device("cpu")
    cuda = device.type == "cuda"
    bufs = [torch.ones(numel, dtype=torch.float32, device=device) for _ in range(parallel)]
    nbytes = numel * 4 * parallel

    def once():
        works = []
        if rank == src:
            works = [dist.isend(b, dst, group=group) for b in bufs]
        elif rank == dst:
            works = [dist.irecv(b, src, group=group) for b in bufs]
        for w in works:
            w.wait()

    for _ in range(warmup):
        once()
    if cuda:
        torch.cuda.synchronize()
    dist.barrier(group=group)
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(trials):
            once()
        b.record()
        torch.cuda.synchronize()
        sec = a.elapsed_time(b) / 1e3 / trials
    else:
        t0 = time.perf_counter()
        for _ in range(trials):
            once()
        sec = (time.perf_counter() - t0) / trials
    t = torch.tensor([sec], dtype=torch.float64, device=device if cuda else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    sec = float(t.item())
    return {"bandwidth_gbs": nbytes / 1e9 / sec, "latency_s": sec / parallel}


def measure_all_pairs_concurrent(numel: int = 64 * 1024 * 1024, warmup: int = 3, trials: int = 5, device=None) -> dict:
    """Every rank sends to rank+1 and receives from rank-1 at the same time (ring shift)."""
    rank, W = dist.get_rank(), dist.get_world_size()
    cuda = device is not None and device.type == "cuda"
    s = torch.ones(numel, dtype=torch.float32, device=device)
    r = torch.empty_like(s)

    def once():
        ops = [dist.P2POp(dist.isend, s, (rank + 1) % W), dist.P2POp(dist.irecv, r, (rank - 1) % W)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()

    for _ in range(warmup):
        once()
    if cuda:
        torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    if cuda:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
    for _ in range(trials):
        once()
    if cuda:
        b.record()
        torch.cuda.synchronize()
        sec = a.elapsed_time(b) / 1e3 / trials
    else:
        sec = (time.perf_counter() - t0) / trials
    t = torch.tensor([sec], dtype=torch.float64, device=device if cuda else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"bandwidth_gbs_per_direction": numel * 4 / 1e9 / float(t.item())}
