"""Layer profiler: times one transformer block's forward and backward on this GPU for
microbatch sizes 1..n and stores the result (with its least-squares line) in
`data/model_latencies.json`, the table the planner reads.

Reference behaviour (utils/runtime_estimator.py:187-414, bench/bench_layer.py): one block,
input = embedding-sized activations in the autocast dtype, 15 timed calls per batch size.
Here time is taken with CUDA events around the calls instead of summing kernel durations
out of a profiler trace, and the block runs through this repository's kernels.
"""
from __future__ import annotations

import json
import statistics
import time
from pathlib import Path
from typing import Optional

import torch

from ..models import registry
from ..ops.api import default_ops_for, get_ops
from ..planner import latency as lat_tbl
from ..utils.metrics import clean_gpu_name


def _time(fn, iters, cuda):
    ts = []
    for _ in range(iters):
        if cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        else:
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(ts)


def profile_block(model_name: str, seq: int, dtype: torch.dtype, batches: int = 4, iters: int = 15, warmup: int = 3,
                  device: Optional[torch.device] = None, ops_name: Optional[str] = None, **overrides) -> dict:
    """{'forward_ms': [...], 'backward_ms': [...], 'activation_bytes': [...]} at microbatch sizes 1..batches."""
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    cuda = device.type == "cuda"
    ops = get_ops(ops_name or default_ops_for(device))
    spec = registry.get_spec(model_name, **overrides)
    blk = registry.make_block(spec)
    _, n = blk.layout()
    flat = torch.empty(n, dtype=torch.float32, device=device)
    blk.init_flat(flat, 1)
    params = flat.to(dtype)
    grads = torch.zeros(n, dtype=torch.float32, device=device)
    blk.bind(params, grads)
    fwd, bwd, act = [], [], []
    for b in range(1, batches + 1):
        T = b * seq
        x = (torch.randn(T, spec.hidden, device=device) * 0.5).to(dtype)
        dy = (torch.randn(T, spec.hidden, device=device) * 0.5).to(dtype)
        ctx = {"B": b, "S": seq}
        sv: dict = {}
        for _ in range(warmup):
            sv = {}
            blk.forward(x, ctx, ops, sv)
            blk.backward(dy, ctx, ops, sv)
        if cuda:
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats(device)
            base = torch.cuda.memory_allocated(device)

        def f():
            nonlocal sv
            sv = {}
            blk.forward(x, ctx, ops, sv)

        fwd.append(_time(f, iters, cuda))
        bwd.append(_time(lambda: blk.backward(dy, ctx, ops, sv), iters, cuda))
        act.append((torch.cuda.max_memory_allocated(device) - base) if cuda else 0)
    return {"forward_ms": fwd, "backward_ms": bwd, "activation_bytes": act}


def profile_chain(model_name: str, seq: int, dtype: torch.dtype, blocks: int = 4, iters: int = 8, warmup: int = 2,
                  device: Optional[torch.device] = None, ops_name: Optional[str] = None, **overrides) -> dict:
    """Times `blocks` consecutive blocks (all forwards, then all backwards, microbatch size 1) against the same
    number of single-block runs: {'chain_ms', 'single_ms', 'overhead'}.  The ratio is what a stage of several
    layers costs beyond the sum of its blocks timed alone (launch gaps, allocator traffic, cold caches between
    different weights); the planner multiplies its block latencies by it."""
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    cuda = device.type == "cuda"
    ops = get_ops(ops_name or default_ops_for(device))
    spec = registry.get_spec(model_name, **overrides)
    blks = []
    for i in range(blocks):
        blk = registry.make_block(spec)
        _, n = blk.layout()
        flat = torch.empty(n, dtype=torch.float32, device=device)
        blk.init_flat(flat, i + 1)
        blk.bind(flat.to(dtype), torch.zeros(n, dtype=torch.float32, device=device))
        blks.append(blk)
    x = (torch.randn(seq, spec.hidden, device=device) * 0.5).to(dtype)
    dy = (torch.randn(seq, spec.hidden, device=device) * 0.5).to(dtype)
    ctx = {"B": 1, "S": seq}

    def chain():
        saved, h = [], x
        for blk in blks:
            sv: dict = {}
            h = blk.forward(h, ctx, ops, sv)
            saved.append(sv)
        g = dy
        for blk, sv in zip(reversed(blks), reversed(saved)):
            g = blk.backward(g, ctx, ops, sv)

    def single():
        for _ in range(blocks):
            sv: dict = {}
            blks[0].forward(x, ctx, ops, sv)
            blks[0].backward(dy, ctx, ops, sv)

    for _ in range(warmup):
        chain()
        single()
    c, s = _time(chain, iters, cuda), _time(single, iters, cuda)
    return {"chain_ms": c, "single_ms": s, "overhead": c / s if s > 0 else 1.0, "blocks": blocks}


def profile_optimizer(n_params: int, shards=(1, 2, 4, 8), device=None, ops_name=None, iters: int = 10) -> dict:
    """Fused Adam time (ms) on a 1/shards slice of a unit (reference utils/runtime_estimator.py:256-279)."""
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    ops = get_ops(ops_name or default_ops_for(device))
    out = {}
    for s in shards:
        n = n_params // s // 8 * 8
        p, m, v = (torch.zeros(n, device=device) for _ in range(3))
        g = torch.zeros(n, device=device)
        p16 = torch.empty(n, dtype=torch.bfloat16, device=device)
        fn = lambda: ops.adam_step(p, m, v, g, p16, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1)
        fn()
        out[str(s)] = _time(fn, iters, device.type == "cuda")
    return out


def profile_and_store(model_name: str, seq: int, dtype_name: str, batches: int = 4, path: Optional[str] = None,
                      device=None, ops_name=None, chain_blocks: int = 0) -> dict:
    from ..config.training_config import dtype_from_str

    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    res = profile_block(model_name, seq, dtype_from_str(dtype_name), batches, device=device, ops_name=ops_name)
    gpu = clean_gpu_name(torch.cuda.get_device_name(device)) if device.type == "cuda" else "cpu"
    p = Path(path) if path else lat_tbl.latencies_path()
    table = lat_tbl.load_table(p)
    lat_tbl.store(table, model_name, gpu, seq, dtype_name, res["forward_ms"], res["backward_ms"])
    if any(res["activation_bytes"]):
        # peak bytes one block adds while it runs forward + backward, per microbatch size: read by the memory model
        lat_tbl.store_activation_bytes(table, model_name, gpu, seq, dtype_name, res["activation_bytes"])
    if chain_blocks > 1:
        ch = profile_chain(model_name, seq, dtype_from_str(dtype_name), chain_blocks, device=device, ops_name=ops_name)
        table.setdefault("_chain_overhead", {}).setdefault(model_name, {})[gpu] = round(ch["overhead"], 4)
        res = {**res, "chain": ch}
    p.parent.mkdir(parents=True, exist_ok=True)
    p.write_text(json.dumps(table, indent=1))
    return {"gpu": gpu, **res}
