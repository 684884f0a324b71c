"""Checkpoint reader with re-sharding: a checkpoint written under one plan (stage split, DP
width, tensor-parallel width) can be loaded under another, because every unit is addressed by its
global id and each rank reads the element ranges of the saved shards that overlap its new shard.
When the tensor-parallel width changes, a block is first put back together from its saved slices
and then cut for the new width."""
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
    for stage, tpi in sorted({(u["stage"], u.get("tp_index", 0)) for u in meta["units"]}):
        units = [u for u in meta["units"] if u["stage"] == stage and u.get("tp_index", 0) == tpi]
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


def _whole_block(directory, meta, offsets, saved: dict, gid: int, which: int, spec, saved_tp: int) -> torch.Tensor:
    """State tensor `which` of block `gid` as the unsplit block lays it out, rebuilt from the saved slices."""
    from ..models import registry

    n = registry.make_block(spec).layout()[1]
    if saved_tp == 1:
        su = saved[(gid, 0)]
        return read_range(directory, meta, offsets, su, which, 0, su["padded"])[:n].clone()
    whole = torch.zeros(n, dtype=torch.float32)
    for t in range(saved_tp):
        su = saved[(gid, t)]
        flat = read_range(directory, meta, offsets, su, which, 0, su["padded"])
        registry.make_block(spec, saved_tp, t).store_into_whole(flat[:su["numel"]], whole)
    return whole


def load_checkpoint(trainer, directory: str) -> int:
    """Loads master weights and Adam state into the trainer's units; returns the saved step."""
    meta = read_meta(directory)
    saved_model = meta["training_config"]["model_name"]
    if saved_model != trainer.cfg.model_name:
        raise CheckpointError(f"checkpoint is for {saved_model}, job trains {trainer.cfg.model_name}")
    saved = {(u["gid"], u.get("tp_index", 0)): u for u in meta["units"]}
    saved_tp = int(meta.get("tensor_parallel_size", 1))
    now_tp, now_t = trainer.cfg.tensor_parallel_size, getattr(trainer, "tp_index", 0)
    offsets = _file_offsets(meta)
    for st in trainer.stages:
        for u in st.engine.units:
            if (u.gid, 0) not in saved:
                raise CheckpointError(f"checkpoint has no unit {u.gid}")
            lo, hi = u.lo, u.hi
            recut = u.layer.kind == "block" and saved_tp != now_tp
            # layers that are not cut (embedding, head) are whole in every slice: read slice 0's copy
            su = saved[(u.gid, now_t if saved_tp == now_tp else 0)]
            if not recut and su["numel"] != u.layer.layout()[1]:
                raise CheckpointError(f"unit {u.gid}: {su['numel']} elements saved, model has {u.layer.layout()[1]}")
            parts = []
            for which in range(3):
                t = torch.zeros(u.shard_n, dtype=torch.float32)
                if recut:
                    whole = _whole_block(directory, meta, offsets, saved, u.gid, which, trainer.spec, saved_tp)
                    if now_tp == 1:
                        mine = whole
                    else:
                        mine = torch.zeros(u.layer.layout()[1], dtype=torch.float32)
                        u.layer.load_from_whole(mine, whole)
                    seg = mine[lo:min(hi, mine.numel())]
                    t[: seg.numel()] = seg
                else:
                    a, b = lo, min(hi, su["padded"])
                    if a < b:
                        t[: b - a] = read_range(directory, meta, offsets, su, which, a, b)
                parts.append(t.to(u.device))
            u.load_state(parts[0], parts[1], parts[2], su.get("step_count", meta["step"]))
    trainer.step_idx = meta["step"]
    trainer.barrier()
    return meta["step"]


def verify_checkpoint(directory: str, values: bool = True) -> dict:
    """Checks a checkpoint directory without a trainer: meta.json readable, every shard file present and exactly as
    long as the unit table says, and (with `values`) every master / moment value finite and every second moment
    non-negative.  Returns a summary; raises CheckpointError at the first structural problem."""
    meta = read_meta(directory)
    offsets = _file_offsets(meta)
    expect: dict = {}
    for u in meta["units"]:
        bd = _bounds(u)
        for idx, r in enumerate(u["shard_ranks"]):
            key = (u["stage"], r)
            expect[key] = expect.get(key, 0) + 3 * (bd[idx + 1] - bd[idx]) * 4
    for (stage, r), size in sorted(expect.items()):
        path = os.path.join(directory, f"stage{stage}_rank{r}.bin")
        if not os.path.exists(path):
            raise CheckpointError(f"missing shard file {path}")
        have = os.path.getsize(path)
        if have != size:
            raise CheckpointError(f"{path} holds {have} bytes, the unit table says {size}"
                                  + (" (truncated)" if have < size else ""))
    out = {"step": meta["step"], "units": len(meta["units"]), "files": len(expect),
           "bytes": sum(expect.values()), "parameters": sum(u["numel"] for u in meta["units"] if u.get("tp_index", 0) == 0
                                                            or meta.get("tensor_parallel_size", 1) > 1),
           "model": meta["training_config"]["model_name"], "bad_units": []}
    if values:
        for u in meta["units"]:
            for which, name in enumerate(("master", "m", "v")):
                t = read_range(directory, meta, offsets, u, which, 0, u["numel"])
                if not bool(torch.isfinite(t).all()) or (name == "v" and bool((t < 0).any())):
                    out["bad_units"].append((u["stage"], u["gid"], u.get("tp_index", 0), name))
    return out


def main(argv=None) -> int:
    """python -m zorse_b200.ckpt.reader <checkpoint directory> [--no-values]"""
    import argparse

    ap = argparse.ArgumentParser(description="verify a checkpoint directory (structure, sizes, finite values)")
    ap.add_argument("directory")
    ap.add_argument("--no-values", action="store_true", help="structure and sizes only")
    a = ap.parse_args(argv)
    try:
        s = verify_checkpoint(a.directory, values=not a.no_values)
    except CheckpointError as e:
        print(f"BAD: {e}")
        return 2
    print(json.dumps(s))
    return 1 if s["bad_units"] else 0


if __name__ == "__main__":
    raise SystemExit(main())
