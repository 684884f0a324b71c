"""Data classes of the planner and readers for its two input files.

`cluster_info.json` (written by the collector) keeps the reference's field names
(example/cluster_info.json; writer utils/collect_cluster_utils.py:110-151): machines with
their GPUs, `gpu_list`, `global_rank_map`, and `bandwidth` with intra-/inter-node bandwidth
(GB/s) and per-message latency.  The collector of this repository adds an optional
`collective_fit` section: per group size R the measured start-up latency and effective
bandwidth of all-gather / reduce-scatter on the NVSwitch domain, and a `units` note.
"""
from __future__ import annotations

import json
from dataclasses import dataclass


@dataclass(frozen=True)
class GPU:
    identifier: str   # cleaned model name, e.g. "b200"
    rank: int
    machine: str = ""
    memory_mib: int = 0


@dataclass
class GPUGroup:
    group_id: int
    gpus: list[GPU]
    all_gather_latency: float = 0.0      # ms, one layer's parameters
    reduce_scatter_latency: float = 0.0  # ms
    send_recv_latency_next: float = 0.0  # ms, one microbatch activation to the next group
    send_recv_latency_prev: float = 0.0
    machines: tuple = ()

    @property
    def ranks(self) -> list[int]:
        return [g.rank for g in self.gpus]


@dataclass
class ModelConfig:
    name: str
    num_layers: int
    hidden_size: int
    parameters_per_layer: int
    total_parameters: int
    sequence_length: int
    global_batch_size: int
    vocab_size: int = 32000


@dataclass
class ModelLatencies:
    """Per-layer forward / backward time (ms) of one microbatch on one GPU model."""
    forward: float
    backward: float

    @property
    def total(self) -> float:
        return self.forward + self.backward


@dataclass
class StagePlan:
    group_id: int
    gpu_ranks: list[int]
    num_microbatches_per_rank: list[int]
    layer_partition: tuple[int, int]

    @property
    def num_layers(self) -> int:
        return self.layer_partition[1] - self.layer_partition[0]


def load_cluster_info(path: str) -> dict:
    with open(path) as f:
        d = json.load(f)
    for k in ("machines", "gpu_list", "bandwidth"):
        if k not in d:
            raise ValueError(f"cluster info file lacks {k!r}")
    return d


def machine_index_of(data: dict, machine: str) -> int:
    for m in data["machines"]:
        if m["machine"] == machine:
            return int(m["machine_index"])
    raise KeyError(machine)


def link_bandwidth(data: dict, g1: dict, g2: dict) -> float:
    """GB/s between two GPUs: the intra-node figure of their machine, or the inter-node figure
    of their machine pair (either orientation)."""
    bw = data["bandwidth"]
    i, j = machine_index_of(data, g1["machine"]), machine_index_of(data, g2["machine"])
    if i == j:
        return float(bw["intranode_bandwidth"][str(i)])
    inter = bw.get("internode_bandwidth", {})
    if str(i) in inter and str(j) in inter[str(i)]:
        return float(inter[str(i)][str(j)])
    return float(inter[str(j)][str(i)])


def link_latency(data: dict, g1: dict, g2: dict) -> float:
    """Seconds per reference message (the collector's 'latency' field) between two GPUs."""
    bw = data["bandwidth"]
    i, j = machine_index_of(data, g1["machine"]), machine_index_of(data, g2["machine"])
    if i == j:
        return float(bw.get("intranode_latency", {}).get(str(i), 0.0))
    inter = bw.get("internode_latency", {})
    if str(i) in inter and str(j) in inter[str(i)]:
        return float(inter[str(i)][str(j)])
    return float(inter.get(str(j), {}).get(str(i), 0.0))
