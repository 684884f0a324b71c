"""torch.profiler integration: Chrome/TensorBoard traces in
`<trace_dir>/<experiment>/GPU_<rank>/` (reference utils/profile.py:51-81,
utils/train_utils.py:224-242), plus helpers that read kernel time back from a trace."""
from __future__ import annotations

import glob
import json
import os

import torch


def first_of_its_model(device_index: int, device_names) -> bool:
    """Whether the device is the first one of its model among the machine's devices (`device_names` in index order)."""
    return list(device_names).index(device_names[device_index]) == device_index


def profiler_context(trace_dir: str, experiment: str, rank: int, detailed: bool = False, unique_gpus_only: bool = False):
    """`unique_gpus_only`: on a machine with several GPUs of one model only the first of them records a trace, the
    others get a context that does nothing (what the reference's trainer does, utils/profile.py:52-63, zorse.py:153)."""
    if unique_gpus_only and torch.cuda.is_available():
        import contextlib

        names = [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())]
        if not first_of_its_model(torch.cuda.current_device(), names):
            return contextlib.nullcontext()
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


def extract_memcpy_runtime(trace_file: str, iterations: int = 1) -> float:
    """Copy-engine time per iteration in ms (reference utils/profile.py:133-158)."""
    return extract_kernel_runtime(trace_file, iterations, cat="gpu_memcpy")


def extract_function_runtime(name: str, trace_file: str, iterations: int = 1, exact: bool = True) -> float:
    """Time per iteration (ms) of the trace events called `name` (any category: a kernel, a CPU operator, a
    `record_function` / NVTX range); `exact=False` matches the name as a substring, which is what kernel names with
    template arguments need (reference utils/profile.py:161-182 matches exactly)."""
    with open(trace_file) as f:
        ev = json.load(f).get("traceEvents", [])
    hit = (lambda n: n == name) if exact else (lambda n: name in n)
    return sum(e.get("dur", 0) for e in ev if hit(str(e.get("name", "")))) / 1e3 / max(iterations, 1)


def fit_line(ys) -> tuple[float, float]:
    """Least-squares (slope, intercept) of ys over x = 1..n, the form in which the layer profiler stores how a
    latency grows with the microbatch size (reference utils/profile.py:124-130); one point gives (y, 0)."""
    ys = [float(y) for y in ys]
    n = len(ys)
    if n == 0:
        raise ValueError("fit_line needs at least one value")
    if n == 1:
        return ys[0], 0.0
    mx, my = (n + 1) / 2.0, sum(ys) / n
    sxx = sum((x - mx) ** 2 for x in range(1, n + 1))
    slope = sum((x - mx) * (y - my) for x, y in zip(range(1, n + 1), ys)) / sxx
    return slope, my - slope * mx


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


# ---- stream classification and overlap accounting ------------------------------------------------
# Reference: utils/train_utils.py:24-221 finds "the" communication and copy streams by kernel name
# (falling back to fixed stream numbers) and charges every idle gap of one stream with the operations
# of another stream that fall into it.  Here every stream is classified, there may be several of a
# kind (two p2p streams, a gather stream, an offload stream), and a gap is charged with the UNION of
# the other kind's busy intervals inside it, so concurrent operations are not counted twice.

COMM_KERNEL_MARKS = ("nccl", "rs_adam", "wait_flags", "peer_pull", "signal", "tp_push", "tp_norm_push", "multimem")
COPY_EVENT_MARKS = ("Memcpy HtoD", "Memcpy DtoH", "Memcpy DtoD")
ALLOC_EVENT_NAMES = ("cudaMalloc", "cudaFree", "cudaMallocAsync", "cudaFreeAsync", "cudaHostAlloc", "cudaFreeHost")


def _stream_of(e):
    return e.get("args", {}).get("stream", e.get("tid"))


def _merge(iv):
    iv = sorted(iv)
    out = []
    for a, b in iv:
        if out and a <= out[-1][1]:
            out[-1][1] = max(out[-1][1], b)
        else:
            out.append([a, b])
    return out


def _overlap(gaps, busy):
    """Total length of the intersection of two sorted lists of disjoint intervals."""
    i = j = 0
    tot = 0.0
    while i < len(gaps) and j < len(busy):
        lo, hi = max(gaps[i][0], busy[j][0]), min(gaps[i][1], busy[j][1])
        if hi > lo:
            tot += hi - lo
        if gaps[i][1] < busy[j][1]:
            i += 1
        else:
            j += 1
    return tot


def classify_streams(events) -> dict:
    """{stream: "compute" | "communication" | "copy"} from what runs on each stream.  A stream is a
    communication stream if most of its time is collective / p2p / fused-collective kernels, a copy
    stream if most of it is memcpy events; every other stream with kernels is a compute stream."""
    t: dict = {}
    for e in events:
        if e.get("cat") not in ("kernel", "gpu_memcpy", "gpu_memset") or e.get("dur", 0) <= 0:
            continue
        s = _stream_of(e)
        d = t.setdefault(s, {"comm": 0.0, "copy": 0.0, "all": 0.0})
        name = e.get("name", "")
        d["all"] += e["dur"]
        if e.get("cat") == "gpu_memcpy" or any(m in name for m in COPY_EVENT_MARKS):
            d["copy"] += e["dur"]
        elif any(m in name.lower() for m in COMM_KERNEL_MARKS):
            d["comm"] += e["dur"]
    out = {}
    for s, d in t.items():
        if d["comm"] > 0.5 * d["all"]:
            out[s] = "communication"
        elif d["copy"] > 0.5 * d["all"]:
            out[s] = "copy"
        else:
            out[s] = "compute"
    return out


def stream_overheads(trace_file: str, gap_threshold_us: float = 0.0, merge_gap_us: float = 500.0) -> dict:
    """Durations per stream kind and the cross-kind overheads (all in ms):

    * `communication_overhead_for_compute`: time inside idle gaps of the compute streams during which
      a communication stream was busy (compute waited while a collective or p2p ran: exposed communication);
    * `copy_overhead_for_compute`: the same for copy streams (offload traffic);
    * `compute_overhead_for_communication`: time inside idle gaps of the communication streams during
      which compute ran (collectives waiting for their inputs);
    * `alloc_overhead_for_compute`: host cudaMalloc / cudaFree calls that fall into compute gaps;
    * `compute_ms` counts gaps shorter than `merge_gap_us` as busy, like the reference's figure.
    """
    with open(trace_file) as f:
        ev = json.load(f).get("traceEvents", [])
    kinds = classify_streams(ev)
    busy = {"compute": [], "communication": [], "copy": []}
    for e in ev:
        if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and e.get("dur", 0) > 0:
            busy[kinds[_stream_of(e)]].append((e["ts"], e["ts"] + e["dur"]))
    alloc = _merge([(e["ts"], e["ts"] + e.get("dur", 0)) for e in ev if e.get("name") in ALLOC_EVENT_NAMES])
    merged = {k: _merge(v) for k, v in busy.items()}

    def gaps(iv):
        return [[a[1], b[0]] for a, b in zip(iv, iv[1:]) if b[0] - a[1] > gap_threshold_us]

    def total(iv):
        return sum(b - a for a, b in iv)

    cg, mg = gaps(merged["compute"]), gaps(merged["communication"])
    compute_ms = total(merged["compute"]) + sum(g[1] - g[0] for g in gaps(merged["compute"]) if g[1] - g[0] < merge_gap_us)
    return {
        "streams": {str(k): v for k, v in kinds.items()},
        "compute_ms": compute_ms / 1e3,
        "communication_ms": total(merged["communication"]) / 1e3,
        "copy_ms": total(merged["copy"]) / 1e3,
        "alloc_ms": total(alloc) / 1e3,
        "communication_overhead_for_compute": _overlap(cg, merged["communication"]) / 1e3,
        "copy_overhead_for_compute": _overlap(cg, merged["copy"]) / 1e3,
        "compute_overhead_for_communication": _overlap(mg, merged["compute"]) / 1e3,
        "alloc_overhead_for_compute": _overlap(cg, alloc) / 1e3,
        "compute_gap_ms": total(cg) / 1e3,
    }
