"""Builds a data set of uneven all-gather / reduce-scatter / broadcast timings over random
shard ratios and message sizes (reference bench/collect_comm_data.py:45-163).

    torchrun --nproc-per-node R -m bench.collect_comm_data --samples 20 --output comm_data.json
"""
import argparse
import json
import random

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--samples", type=int, default=20)
    ap.add_argument("--min_mb", type=float, default=1.0)
    ap.add_argument("--max_mb", type=float, default=1000.0)
    ap.add_argument("--output", default="comm_data.json")
    ap.add_argument("--backend", default=None)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    from zorse_b200.parallel.groups import dist_init
    from zorse_b200.profiler.collectives import (AllGather, Broadcast, ReduceScatter, UnevenAllGather,
                                                 UnevenReduceScatter, time_pattern)

    dev = dist_init(a.backend)
    R = dist.get_world_size()
    rng = random.Random(a.seed)  # same seed on every rank: identical sizes and ratios
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    rows = []
    for _ in range(a.samples):
        mb = 10 ** rng.uniform(torch.log10(torch.tensor(a.min_mb)).item(), torch.log10(torch.tensor(a.max_mb)).item())
        numel = int(mb * 2**20 / (2 if dt == torch.bfloat16 else 4))
        ratios = [rng.uniform(0.2, 1.0) for _ in range(R)]
        for pat in (AllGather(numel, dt, device=dev), ReduceScatter(numel, dt, device=dev), Broadcast(numel, dt, device=dev),
                    UnevenAllGather(numel, ratios, dt, device=dev), UnevenReduceScatter(numel, ratios, dt, device=dev)):
            r = time_pattern(pat, warmup=2, trials=5)
            rows.append({"pattern": pat.name, "size_mb": mb, "ratios": ratios if "uneven" in pat.name else None, **r})
    if dist.get_rank() == 0:
        with open(a.output, "w") as f:
            json.dump(rows, f, indent=1)
        print(f"wrote {len(rows)} rows to {a.output}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
