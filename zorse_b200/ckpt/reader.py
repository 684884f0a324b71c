"""Checkpoint reader with re-sharding: a checkpoint written under one plan (stage split, DP
width) can be loaded under another, because every unit is addressed by its global id and
each rank reads the element ranges of the saved shards that overlap its new shard."""
from __future__ import annotations

import json
import os

import numpy as np
import torch


class CheckpointError(RuntimeError):
    pass


def read_meta(directory: str) -> dict:
    p = os.path.join(directory, "meta.json")
    if not os.path.exists(p):
        raise CheckpointError(f"{directory} has no meta.json (incomplete or not a checkpoint)")
    with open(p) as f:
        meta = json.load(f)
    if meta.get("format_version") != 1:
        raise CheckpointError(f"unsupported checkpoint format {meta.get('format_version')}")
    return meta


def _bounds(unit: dict) -> list[int]:
    """Element offsets of the saved shards (files written before unequal shards existed carry
    only the common shard size)."""
    if "shard_offsets" in unit:
        return list(unit["shard_offsets"])
    return [i * unit["shard_numel"] for i in range(len(unit["shard_ranks"]) + 1)]


def _file_offsets(meta: dict) -> dict:
    """(stage, rank) -> {gid: byte offset of the unit's (master, m, v) block in that file}."""
    out: dict = {}
    for stage in sorted({u["stage"] for u in meta["units"]}):
        units = [u for u in meta["units"] if u["stage"] == stage]
        for idx, r in enumerate(units[0]["shard_ranks"]):
            off, table = 0, {}
            for u in units:
                table[u["gid"]] = off
                bd = _bounds(u)
                off += 3 * (bd[idx + 1] - bd[idx]) * 4
            out[(stage, r)] = table
    return out


def read_range(directory: str, meta: dict, offsets: dict, unit: dict, which: int, lo: int, hi: int) -> torch.Tensor:
    """Elements [lo, hi) of the padded flat tensor `which` (0 master, 1 m, 2 v) of a saved unit."""
    out = torch.zeros(hi - lo, dtype=torch.float32)
    bd = _bounds(unit)
    for idx, r in enumerate(unit["shard_ranks"]):
        s0, sn = bd[idx], bd[idx + 1] - bd[idx]
        a, b = max(lo, s0), min(hi, s0 + sn)
        if a >= b:
            continue
        path = os.path.join(directory, f"stage{unit['stage']}_rank{r}.bin")
        if not os.path.exists(path):
            raise CheckpointError(f"missing shard file {path}")
        need = offsets[(unit["stage"], r)][unit["gid"]] + (which * sn + (b - s0)) * 4
        if os.path.getsize(path) < need:
            raise CheckpointError(f"{path} is truncated ({os.path.getsize(path)} bytes, need {need})")
        start = offsets[(unit["stage"], r)][unit["gid"]] + (which * sn + (a - s0)) * 4
        arr = np.fromfile(path, dtype="<f4", count=b - a, offset=start)
        out[a - lo:b - lo] = torch.from_numpy(arr.copy())
    return out


def load_checkpoint(trainer, directory: str) -> int:
    """Loads master weights and Adam state into the trainer's units; returns the saved step."""
    meta = read_meta(directory)
    saved_model = meta["training_config"]["model_name"]
    if saved_model != trainer.cfg.model_name:
        raise CheckpointError(f"checkpoint is for {saved_model}, job trains {trainer.cfg.model_name}")
    by_gid = {u["gid"]: u for u in meta["units"]}
    offsets = _file_offsets(meta)
    for st in trainer.stages:
        for u in st.engine.units:
            if u.gid not in by_gid:
                raise CheckpointError(f"checkpoint has no unit {u.gid}")
            su = by_gid[u.gid]
            if su["numel"] != u.layer.layout()[1]:
                raise CheckpointError(f"unit {u.gid}: {su['numel']} elements saved, model has {u.layer.layout()[1]}")
            lo, hi = u.lo, u.hi
            parts = []
            for which in range(3):
                t = torch.zeros(u.shard_n, dtype=torch.float32)
                a, b = lo, min(hi, su["padded"])
                if a < b:
                    t[: b - a] = read_range(directory, meta, offsets, su, which, a, b)
                parts.append(t.to(u.device))
            u.load_state(parts[0], parts[1], parts[2], su.get("step_count", meta["step"]))
    trainer.step_idx = meta["step"]
    trainer.barrier()
    return meta["step"]
