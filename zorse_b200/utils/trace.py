"""torch.profiler integration: Chrome/TensorBoard traces in
`<trace_dir>/<experiment>/GPU_<rank>/` (reference utils/profile.py:51-81,
utils/train_utils.py:224-242), plus helpers that read kernel time back from a trace."""
from __future__ import annotations

import glob
import json
import os

import torch


def profiler_context(trace_dir: str, experiment: str, rank: int, detailed: bool = False):
    out = os.path.join(os.path.expanduser(trace_dir), experiment, f"GPU_{rank}")
    os.makedirs(out, exist_ok=True)
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    return torch.profiler.profile(activities=acts, on_trace_ready=torch.profiler.tensorboard_trace_handler(out),
                                  record_shapes=detailed, profile_memory=detailed, with_stack=detailed)


def newest_trace(path: str):
    files = glob.glob(os.path.join(path, "**", "*.json"), recursive=True)
    return max(files, key=os.path.getmtime) if files else None


def extract_kernel_runtime(trace_file: str, iterations: int = 1, cat: str = "kernel") -> float:
    """Sum of the durations (ms) of events of category `cat` divided by `iterations`."""
    with open(trace_file) as f:
        ev = json.load(f).get("traceEvents", [])
    return sum(e.get("dur", 0) for e in ev if e.get("cat") == cat) / 1e3 / max(iterations, 1)


def stream_busy_and_gaps(trace_file: str, gap_threshold_us: float = 0.0) -> dict:
    """Per CUDA stream: busy time and idle gaps between consecutive kernels (ms)."""
    with open(trace_file) as f:
        ev = [e for e in json.load(f).get("traceEvents", []) if e.get("cat") in ("kernel", "gpu_memcpy")]
    out: dict = {}
    by = {}
    for e in ev:
        by.setdefault(e.get("args", {}).get("stream", e.get("tid")), []).append(e)
    for s, es in by.items():
        es.sort(key=lambda e: e["ts"])
        busy = sum(e["dur"] for e in es)
        gaps = sum(max(0.0, b["ts"] - (a["ts"] + a["dur"])) for a, b in zip(es, es[1:])
                   if b["ts"] - (a["ts"] + a["dur"]) > gap_threshold_us)
        out[s] = {"busy_ms": busy / 1e3, "gap_ms": gaps / 1e3, "kernels": len(es)}
    return out
