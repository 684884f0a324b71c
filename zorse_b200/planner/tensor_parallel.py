"""Planning with tensor-parallel lanes.

With `tensor_parallel_size = t` the trainer's rank numbers name lanes of t processes.  The planner
handles that by planning for the lanes: `coarsen()` merges every t consecutive GPUs of a machine
(same GPU model) into one lane that has t times the memory, and `lane_latencies()` turns the
profiled per-layer compute latencies into lane latencies: compute divided by t, plus the lane's
collectives on [tokens, hidden] activations (forward: two all-gathers and two reduce-scatters per
block; backward: four all-gathers and two reduce-scatters, as `models/tp_layers.py` issues them),
costed with the same communication model the planner uses for ZeRO.  The model is not calibrated
against measurements yet; `efficiency` scales the compute term for the smaller GEMMs of a slice.
"""
from __future__ import annotations

import copy

from ..utils.metrics import clean_gpu_name
from . import comm_model

FWD_GATHERS, FWD_SCATTERS, BWD_GATHERS, BWD_SCATTERS = 2, 2, 4, 2


def coarsen(data: dict, t: int) -> tuple[dict, dict]:
    """(cluster description whose "GPUs" are lanes of t GPUs, {lane rank: original global ranks})."""
    if t <= 1:
        return data, {int(g["global_rank"]): [int(g["global_rank"])] for g in data["gpu_list"]}
    out = copy.deepcopy(data)
    lanes, members = [], {}
    for m in out["machines"]:
        gpus = sorted((g for g in out["gpu_list"] if g.get("machine") == m.get("machine")), key=lambda g: int(g["index"]))
        if len(gpus) % t:
            raise ValueError(f"machine {m.get('machine')}: {len(gpus)} GPUs do not form lanes of {t}")
        m_lanes = []
        for i in range(0, len(gpus), t):
            grp = gpus[i:i + t]
            if len({clean_gpu_name(g["name"]) for g in grp}) != 1:
                raise ValueError(f"machine {m.get('machine')}: GPUs {[g['index'] for g in grp]} of one lane differ in model")
            lane = dict(grp[0])
            lane["global_rank"] = len(lanes)
            lane["id"] = f"gpu_{lane['global_rank']}"
            lane["index"] = i // t
            lane["memory_total_mib"] = sum(int(g.get("memory_total_mib", 0)) for g in grp)
            members[lane["global_rank"]] = [int(g["global_rank"]) for g in grp]
            lanes.append(lane)
            m_lanes.append(lane)
        m["gpus"], m["num_gpus"] = m_lanes, len(m_lanes)
    out["gpu_list"], out["total_gpus"] = lanes, len(lanes)
    if "global_rank_map" in out:
        out["global_rank_map"] = {str(g["global_rank"]): {"machine": g.get("machine"), "local_rank": g["index"],
                                                          "machine_index": next((m.get("machine_index", 0) for m in out["machines"]
                                                                                 if m.get("machine") == g.get("machine")), 0)}
                                  for g in lanes}
    return out, members


def lane_collective_ms(data: dict, ranks, tokens: int, hidden: int, dtype_bytes: int) -> tuple[float, float]:
    """(forward, backward) milliseconds of one block's lane collectives for one microbatch."""
    size = float(tokens) * hidden * dtype_bytes
    ag = comm_model.collective_ms(data, ranks, size, "all_gather")
    rs = comm_model.collective_ms(data, ranks, size, "reduce_scatter")
    return FWD_GATHERS * ag + FWD_SCATTERS * rs, BWD_GATHERS * ag + BWD_SCATTERS * rs


def lane_latencies(lat_tbl: dict, t: int, comm_fwd_ms: float, comm_bwd_ms: float, efficiency: float = 0.92) -> dict:
    """Per-"GPU" (lane) block latencies from the profiled single-GPU ones."""
    if t <= 1:
        return lat_tbl
    return {g: type(v)(v.forward / t / efficiency + comm_fwd_ms, v.backward / t / efficiency + comm_bwd_ms)
            for g, v in lat_tbl.items()}
