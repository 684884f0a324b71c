"""Restart after a failure: newest complete checkpoint + a plan for the GPUs that are left.

    python -m zorse_b200.cli.recover --checkpoint_dir ck --cluster_info_file cluster_info.json \
        [--exclude_ranks 3,5] [--output training_config.json]

The trainer's watchdog ends a stuck job with the names of the silent ranks; this tool is the step
after it.  It picks the newest checkpoint directory that is complete (`meta.json` is written
last), takes the model, batch, sequence length and dtypes from it, removes the failed GPUs from
the cluster description (renumbering the rest), runs the planner on what is left and writes the
new training config.  The checkpoint reader re-shards, so the job resumes under the new plan with
`zorse.py --config_file <output> --resume <checkpoint>`; the command is printed.

There is no in-place elastic resizing: a changed world is a new job that starts from a
checkpoint.  (The reference has neither checkpoints nor recovery.)
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import re
import sys
from typing import Optional


def latest_checkpoint(directory: str, verify: bool = False) -> Optional[str]:
    """Path of the `step_<n>` sub-directory with the largest n that holds a meta.json; with `verify` also one whose
    shard files are all there and as long as its unit table says (a newer but damaged checkpoint is passed over)."""
    if not os.path.isdir(directory):
        return None
    found = []
    for name in os.listdir(directory):
        m = re.fullmatch(r"step_(\d+)", name)
        p = os.path.join(directory, name)
        if m and os.path.exists(os.path.join(p, "meta.json")):
            found.append((int(m.group(1)), p))
    for _, p in sorted(found, reverse=True):
        if not verify:
            return p
        from ..ckpt.reader import CheckpointError, verify_checkpoint

        try:
            verify_checkpoint(p, values=False)
            return p
        except (CheckpointError, OSError, ValueError, KeyError):
            continue
    return None


def shrink_cluster(data: dict, exclude_ranks) -> dict:
    """Cluster description without the GPUs whose global rank is in `exclude_ranks`; the remaining
    GPUs are renumbered 0 .. n-1 in their old order, machines left without a GPU are dropped."""
    gone = set(int(r) for r in exclude_ranks)
    out = copy.deepcopy(data)
    known = {int(g["global_rank"]) for g in data["gpu_list"]}
    if gone - known:
        raise ValueError(f"ranks {sorted(gone - known)} are not in the cluster description")
    keep = [g for g in out["gpu_list"] if int(g["global_rank"]) not in gone]
    if not keep:
        raise ValueError("no GPU would be left")
    renum = {int(g["global_rank"]): i for i, g in enumerate(keep)}
    for g in keep:
        g["global_rank"] = renum[int(g["global_rank"])]
        if "id" in g:
            g["id"] = f"gpu_{g['global_rank']}"
    out["gpu_list"] = keep
    out["total_gpus"] = len(keep)
    machines = []
    for m in out.get("machines", []):
        gpus = [g for g in keep if g.get("machine") == m.get("machine")]
        if gpus:
            m = dict(m, gpus=gpus, num_gpus=len(gpus))
            machines.append(m)
    out["machines"] = machines
    if "global_rank_map" in out:
        out["global_rank_map"] = {str(g["global_rank"]): {"machine": g.get("machine"), "local_rank": g.get("index"),
                                                          "machine_index": next((m.get("machine_index", 0) for m in machines
                                                                                 if m.get("machine") == g.get("machine")), 0)}
                                  for g in keep}
    return out


def replan(meta: dict, cluster: dict, **plan_kw) -> dict:
    """Training config (dictionary) for the job described by a checkpoint's meta on `cluster`."""
    from ..planner.plan import export_config, plan

    tc = meta["training_config"]
    # keep the old job's tensor-parallel width while the remaining GPUs still form whole lanes; otherwise plan
    # without it (the checkpoint reader re-cuts the blocks for any width)
    tp = int(tc.get("tensor_parallel_size", 1))
    if tp > 1:
        per_machine = {}
        for g in cluster["gpu_list"]:
            per_machine[g.get("machine")] = per_machine.get(g.get("machine"), 0) + 1
        if any(n % tp for n in per_machine.values()):
            tp = 1
    best, _ = plan(cluster, tc["model_name"], global_batch_size=int(tc["global_batch_size"]),
                   sequence_length=int(tc["sequence_length"]), tensor_parallel_size=tp, **plan_kw)
    if best is None:
        raise RuntimeError("the planner found no plan that fits the remaining GPUs")
    d = export_config(best, tc["model_name"], int(tc["global_batch_size"]), int(tc["sequence_length"]),
                      int(tc.get("vocab_size", 32000)), tc.get("autocast_dtype", "bfloat16"),
                      tc.get("reduce_dtype", "float32"), total_ranks=cluster["total_gpus"] // tp,
                      tensor_parallel_size=tp)
    for k in ("schedule", "grad_norm_compat", "activation_recompute", "activation_offload"):
        if k in tc and k not in d:
            d[k] = tc[k]      # choices of the old job that do not depend on the layout
    return d


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--checkpoint_dir", required=True)
    ap.add_argument("--cluster_info_file", required=True)
    ap.add_argument("--exclude_ranks", default="", help="comma-separated global ranks of the GPUs that failed")
    ap.add_argument("--output", default="training_config.json")
    a = ap.parse_args(argv)
    from ..ckpt.reader import read_meta

    ck = latest_checkpoint(a.checkpoint_dir)
    if ck is None:
        sys.stderr.write(f"no complete checkpoint under {a.checkpoint_dir}\n")
        return 2
    meta = read_meta(ck)
    with open(a.cluster_info_file) as f:
        cluster = json.load(f)
    gone = [int(x) for x in a.exclude_ranks.split(",") if x.strip()]
    if gone:
        cluster = shrink_cluster(cluster, gone)
    cfg = replan(meta, cluster)
    with open(a.output, "w") as f:
        json.dump(cfg, f, indent=1)
    n = cluster["total_gpus"]
    from ..config.training_config import parse_pipeline_dict

    n = min(n, parse_pipeline_dict(cfg).world_size)
    print(f"checkpoint {ck} (step {meta['step']}), {n} GPUs left, plan written to {a.output}")
    print(f"python -m torch.distributed.run --nproc-per-node {n} zorse.py --config_file {a.output} --resume {ck}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
