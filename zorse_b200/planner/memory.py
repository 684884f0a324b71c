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
                       dtype_multiplier: float = 2.0, optimizer_multiplier: float = 12.0,
                       block_activation_bytes: float | None = None) -> float:
    """`block_activation_bytes`: measured peak of one block's forward + backward at this microbatch size (layer
    profiler); when given it replaces the closed-form `2 * mbs * S * H * dm` live-activation term."""
    Lg = sum(layers_per_stage)
    if len(layers_per_stage) == 1:
        maxpair = layers_per_stage[0]
    else:
        maxpair = max(max(a + b for a, b in zip(layers_per_stage, layers_per_stage[1:])), layers_per_stage[0])
    P, dm, om, N = params_per_layer, dtype_multiplier, optimizer_multiplier, n_gpus
    act = mbs * seq * hidden * dm
    live = 2 * act if block_activation_bytes is None else float(block_activation_bytes)
    return P * dm * maxpair + P * dm * (Lg - maxpair) / N + live + P * om * Lg / N + act


def estimate_memory_usage(total_params: int, num_layers: int, hidden: int, seq: int, mbs: int, num_shards: int = 1,
                          block_activation_bytes: float | None = None, recompute: bool = True,
                          dtype_multiplier: float = 2.0) -> dict:
    """Whole-model estimate in GiB with the reference's terms (utils/runtime_estimator.py:108-184): activations of
    the block being (re)computed, one checkpoint (block input) per layer and microbatch, and the training state
    (16 bytes per parameter: fp32 parameters, gradients and two moments) over the shards.  Without recomputation
    every layer keeps its activations."""
    GiB = 1024 ** 3
    ckpt_one = mbs * seq * hidden * dtype_multiplier
    act_one = block_activation_bytes if block_activation_bytes is not None else 2 * ckpt_one
    activation = act_one if recompute else act_one * num_layers
    checkpoints = ckpt_one * num_layers if recompute else 0.0
    state = 16.0 * total_params / max(num_shards, 1)
    return {"activation_gib": activation / GiB, "checkpoint_gib": checkpoints / GiB, "training_state_gib": state / GiB,
            "total_gib": (activation + checkpoints + state) / GiB}


def validate_memory(stages, groups, model, mbs: int, dtype_multiplier: float = 2.0, optimizer_multiplier: float = 12.0,
                    reserved_gb: float = 2.0, table: dict | None = None, dtype: str = "bfloat16") -> tuple[bool, dict]:
    """stages: list of StagePlan; groups: {group_id: GPUGroup}. Returns (fits, per-group GB).  With a profile
    `table` that holds measured activation bytes for the model on a group's GPUs, the measured figure is used."""
    from .latency import activation_bytes

    per_group: dict[int, list[int]] = {}
    for st in stages:
        per_group.setdefault(st.group_id, []).append(st.num_layers)
    used, ok = {}, True
    for gid, layers in per_group.items():
        grp = groups[gid]
        measured = None
        if table:
            ms = [activation_bytes(table, model.name, g.identifier, model.sequence_length, dtype, mbs) for g in grp.gpus]
            if all(m is not None for m in ms):
                measured = max(ms)
        b = group_memory_bytes(layers, len(grp.gpus), model.parameters_per_layer, mbs, model.sequence_length,
                               model.hidden_size, dtype_multiplier, optimizer_multiplier, block_activation_bytes=measured)
        gb = b / 1e9 + reserved_gb
        limit = min(GPU_MEMORY_GB.get(g.identifier, g.memory_mib / 1024.0 if g.memory_mib else 16.0) for g in grp.gpus)
        used[gid] = gb
        ok = ok and gb <= limit
    return ok, used
