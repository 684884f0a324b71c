"""Memory model of a plan (reference zorse_optimizer/utils.py:11-116).

Per group, bytes =
    P*dm*maxpair                      unsharded parameters of the layers that may be gathered at once
  + P*dm*(Lg - maxpair)/N             the remaining layers, sharded
  + 2*mbs*S*H*dm                      live activations
  + P*om*Lg/N                         fp32 master + Adam moments, sharded
  + mbs*S*H*dm                        one p2p buffer
  + reserved
against the smallest GPU of the group.  P = parameters per layer, dm = dtype multiplier (2),
om = optimizer multiplier (12), N = GPUs of the group, Lg = layers the group owns over all its
stages, maxpair = largest layer count of two consecutive local stages (or of the first stage).
Embedding / head parameters are not counted (as in the reference).
"""
from __future__ import annotations

GPU_MEMORY_GB = {"b200": 178.0, "h100-nvl": 94.0, "h100": 80.0, "a100x80": 80.0, "a100": 40.0, "l40s": 48.0,
                 "a6000": 47.99, "l4": 22.5, "a10g": 24.0, "v100": 32.0, "t4": 16.0, "p40": 24.0}


def group_memory_bytes(layers_per_stage: list[int], n_gpus: int, params_per_layer: int, mbs: int, seq: int, hidden: int,
                       dtype_multiplier: float = 2.0, optimizer_multiplier: float = 12.0) -> float:
    Lg = sum(layers_per_stage)
    if len(layers_per_stage) == 1:
        maxpair = layers_per_stage[0]
    else:
        maxpair = max(max(a + b for a, b in zip(layers_per_stage, layers_per_stage[1:])), layers_per_stage[0])
    P, dm, om, N = params_per_layer, dtype_multiplier, optimizer_multiplier, n_gpus
    act = mbs * seq * hidden * dm
    return P * dm * maxpair + P * dm * (Lg - maxpair) / N + 2 * act + P * om * Lg / N + act


def validate_memory(stages, groups, model, mbs: int, dtype_multiplier: float = 2.0, optimizer_multiplier: float = 12.0,
                    reserved_gb: float = 2.0) -> tuple[bool, dict]:
    """stages: list of StagePlan; groups: {group_id: GPUGroup}. Returns (fits, per-group GB)."""
    per_group: dict[int, list[int]] = {}
    for st in stages:
        per_group.setdefault(st.group_id, []).append(st.num_layers)
    used, ok = {}, True
    for gid, layers in per_group.items():
        grp = groups[gid]
        b = group_memory_bytes(layers, len(grp.gpus), model.parameters_per_layer, mbs, model.sequence_length,
                               model.hidden_size, dtype_multiplier, optimizer_multiplier)
        gb = b / 1e9 + reserved_gb
        limit = min(GPU_MEMORY_GB.get(g.identifier, g.memory_mib / 1024.0 if g.memory_mib else 16.0) for g in grp.gpus)
        used[gid] = gb
        ok = ok and gb <= limit
    return ok, used
