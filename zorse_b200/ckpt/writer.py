"""Checkpoint writer (the reference has no checkpointing at all; this format is new).

Layout: `<dir>/step_<n>/meta.json` + one flat binary per (stage, rank) `stage<s>_rank<r>.bin`.
`meta.json` holds the training config, the step, seeds, dtypes and, per stage, the unit table:
global unit id, kind, unpadded and padded element counts, shard-group ranks and the element
offsets of their shards (equal or, with `shard_ratio`, unequal) and, with tensor parallelism, which
slice of the layer the entry is (`tp_index`; ranks are process ranks).  A rank file is the concatenation, per unit in table order, of the fp32 master
shard, Adam m and v shards (little-endian float32).  Files are written to a temporary name,
fsynced and renamed, `meta.json` last, so a directory with a `meta.json` is complete.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from ..config.training_config import to_dict

FORMAT_VERSION = 1


def _atomic_write(path: str, data: bytes) -> None:
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def unit_table(trainer) -> list[dict]:
    """Describes every unit of every local stage (identical on all ranks of a stage)."""
    out = []
    for st in trainer.stages:
        for u in st.engine.units:
            out.append({"stage": st.stage_id, "gid": u.gid, "kind": u.layer.kind, "numel": u.layer.layout()[1],
                        "padded": u.n, "shard_ranks": list(u.shard_group.ranks), "shard_numel": u.shard_n,
                        "shard_offsets": list(u.offs), "step_count": u.step_count,
                        "tp_index": getattr(trainer, "tp_index", 0)})
    return out


def save_checkpoint(trainer, directory: str, step: int) -> str:
    d = os.path.join(directory, f"step_{step}")
    os.makedirs(d, exist_ok=True)
    trainer.synchronize()
    for st in trainer.stages:
        chunks = []
        for u in st.engine.units:
            for t in u.state_tensors().values():
                chunks.append(t.detach().to("cpu", torch.float32).contiguous().numpy().tobytes())
        _atomic_write(os.path.join(d, f"stage{st.stage_id}_rank{trainer.rank}.bin"), b"".join(chunks))
    tables = [None] * trainer.world
    if dist.is_available() and dist.is_initialized():
        grp = trainer.gloo_group
        if grp is not None or dist.get_backend() == "gloo":
            dist.all_gather_object(tables, unit_table(trainer), group=grp)
        else:
            tables = [unit_table(trainer)]
        trainer.barrier()
    else:
        tables = [unit_table(trainer)]
    if trainer.rank == 0:
        seen, units = set(), []
        for tb in tables:
            for e in tb or []:
                key = (e["stage"], e["gid"], e.get("tp_index", 0))
                if key not in seen:
                    seen.add(key)
                    units.append(e)
        meta = {"format_version": FORMAT_VERSION, "step": step, "seed": trainer.opt.seed,
                "training_config": to_dict(trainer.cfg), "compute_dtype": trainer.cfg.autocast_dtype,
                "world_size": trainer.world, "tensor_parallel_size": trainer.cfg.tensor_parallel_size,
                "units": sorted(units, key=lambda e: (e["stage"], e["gid"], e.get("tp_index", 0)))}
        _atomic_write(os.path.join(d, "meta.json"), json.dumps(meta, indent=1).encode())
    trainer.barrier()
    return d
