"""torchrun worker: all-gather and reduce-scatter of one layer's parameters on the GPUs it is
launched on.  The reference's planner launches a script of this name over ssh
(zorse_optimizer/profiler.py:199, 290) but does not ship it; the output schema is the one of
its sample result (zorse_optimizer/results/profile_results_0.json): avg/min/max/std times in
ms and bandwidth in MB/s for both collectives.

    torchrun --nproc-per-node 4 -m zorse_b200.profiler.run_comm_profiling --num_parameters 202383360 \
        --dtype bfloat16 --num_trials 10 --num_warmup 3 --output profile_results.json [--fit]
"""
from __future__ import annotations

import argparse
import json

import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--num_parameters", type=int, required=True)
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--num_trials", type=int, default=10)
    ap.add_argument("--num_warmup", type=int, default=3)
    ap.add_argument("--output", default="profile_results.json")
    ap.add_argument("--fit", action="store_true", help="also time 1/16, 1/4 and 1x the size and fit alpha/bandwidth")
    ap.add_argument("--backend", default=None)
    a = ap.parse_args(argv)
    from ..config.training_config import dtype_from_str
    from ..parallel.groups import dist_init
    from .collectives import AllGather, ReduceScatter, fit_switch_model, time_pattern

    dev = dist_init(a.backend)
    dt = dtype_from_str(a.dtype)
    res = {"profile_results": {}}
    for cls in (AllGather, ReduceScatter):
        res["profile_results"][cls.name] = time_pattern(cls(a.num_parameters, dt, device=dev), a.num_warmup, a.num_trials)
    if a.fit:
        R = dist.get_world_size()
        res["fit"] = {}
        for cls in (AllGather, ReduceScatter):
            sizes, times = [], []
            for frac in (16, 4, 1):
                p = cls(max(a.num_parameters // frac, R * 64), dt, device=dev)
                sizes.append(p.bytes())
                times.append(time_pattern(p, a.num_warmup, a.num_trials)["min_time_ms"])
            res["fit"][cls.name] = {str(R): fit_switch_model(sizes, times, R)}
    if dist.get_rank() == 0:
        with open(a.output, "w") as f:
            json.dump(res, f, indent=1)
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
