"""Collective and point-to-point cost models (milliseconds, GB/s, bytes throughout).

Two families:
* the reference's ring-on-the-slowest-link estimates (comm_model.py:67-114): used for
  multi-node inputs and whenever the cluster file has no measured fit;
* the NVSwitch fit `t = alpha(R) + (R-1)/R * bytes / BW(R)` with alpha and BW measured per
  group size by this repository's collector — on one NVSwitch domain every GPU reaches every
  peer at full bandwidth, so the one-shot (direct) algorithms the fused kernels use move
  (R-1)/R of the message per rank with a single latency term and no ring.
"""
from __future__ import annotations

from typing import Sequence

from .cluster import link_bandwidth

DTYPE_BYTES = {"float16": 2, "bfloat16": 2, "float32": 4}
RING_FUDGE = 1.15


def tensor_size_bytes(parameters_per_layer: int, dtype: str) -> float:
    return float(parameters_per_layer) * DTYPE_BYTES[dtype]


def tensor_size_gb(parameters_per_layer: int, dtype: str) -> float:
    return tensor_size_bytes(parameters_per_layer, dtype) / 1e9


def bandwidth_matrix(data: dict, ranks: Sequence[int]) -> list[list[float]]:
    by_rank = {g["global_rank"]: g for g in data["gpu_list"]}
    n = len(ranks)
    m = [[0.0] * n for _ in range(n)]
    for i in range(n):
        for j in range(n):
            if i != j:
                m[i][j] = link_bandwidth(data, by_rank[ranks[i]], by_rank[ranks[j]])
    return m


def ring_collective_ms(size_bytes: float, bw: list[list[float]]) -> float:
    """(n-1)/n of the message over the slowest link of the ring 0->1->...->n-1->0."""
    n = len(bw)
    if n <= 1:
        return 0.0
    slow = min(bw[i][(i + 1) % n] for i in range(n))
    return (n - 1) / n * size_bytes / 1e9 / slow * 1e3


def ring_collective_ms_v2(size_bytes: float, bw: list[list[float]]) -> float:
    """Sum over the n-1 ring steps of the slowest hop moving one n-th of the message, x 1.15."""
    n = len(bw)
    if n <= 1:
        return 0.0
    per_step = max((size_bytes / n) / 1e9 / bw[i][(i + 1) % n] for i in range(n)) * 1e3
    return RING_FUDGE * (n - 1) * per_step


def switch_collective_ms(size_bytes: float, R: int, alpha_ms: float, bw_gbs: float) -> float:
    if R <= 1:
        return 0.0
    return alpha_ms + (R - 1) / R * size_bytes / 1e9 / bw_gbs * 1e3


def collective_ms(data: dict, ranks: Sequence[int], size_bytes: float, kind: str = "all_gather") -> float:
    """All-gather / reduce-scatter time of `size_bytes` over `ranks`: the measured NVSwitch fit
    when the ranks share a machine and the cluster file has one, else the ring model."""
    R = len(ranks)
    if R <= 1:
        return 0.0
    fit = data.get("collective_fit", {}).get(kind, {}).get(str(R))
    by_rank = {g["global_rank"]: g for g in data["gpu_list"]}
    same_machine = len({by_rank[r]["machine"] for r in ranks}) == 1
    if fit and same_machine:
        return switch_collective_ms(size_bytes, R, float(fit["alpha_ms"]), float(fit["bandwidth_gbs"]))
    return ring_collective_ms_v2(size_bytes, bandwidth_matrix(data, ranks))


def p2p_ms(size_bytes: float, bw_gbs: float, ref_latency_s: float, ref_bytes: float = 1e7) -> float:
    """Send/recv time of one message over a link whose `ref_bytes` message was measured at
    `ref_latency_s`: below the reference size the time shrinks towards 80 % of the reference,
    above it the excess bytes move at link bandwidth (reference zorse_planner.py:251-352)."""
    ref_ms = ref_latency_s * 1e3
    if ref_ms <= 0.0:
        return size_bytes / 1e9 / bw_gbs * 1e3
    if size_bytes <= ref_bytes:
        return ref_ms * (0.8 + 0.2 * size_bytes / ref_bytes)
    return ref_ms + (size_bytes - ref_bytes) / 1e9 / bw_gbs * 1e3
