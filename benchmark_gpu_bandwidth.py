#!/usr/bin/env python
"""torchrun worker of the cluster collector (reference benchmark_gpu_bandwidth.py).

  --intranode : NCCL between GPU pairs of this machine (GPU 0 <-> 1 with --fast_intra, else
                the minimum over all pairs), plus the all-links-at-once ring shift
  --internode : Gloo on CPU tensors between the first ranks of two nodes
Prints "Bandwidth: x GB/s" and "Latency: x s" (per message) and writes a JSON result file.
"""
import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--intranode", action="store_true")
    ap.add_argument("--internode", action="store_true")
    ap.add_argument("--fast_intra", action="store_true")
    ap.add_argument("--send_msg_size", type=int, default=10_000_000, help="float32 elements per message")
    ap.add_argument("--parallel", type=int, default=1)
    ap.add_argument("--num_trials", type=int, default=10)
    ap.add_argument("--num_warmup", type=int, default=5)
    ap.add_argument("--output_dir", default="results")
    ap.add_argument("--machine_index", type=int, default=0)
    a = ap.parse_args(argv)
    import torch
    import torch.distributed as dist

    from zorse_b200.parallel.groups import dist_init
    from zorse_b200.profiler.bandwidth import measure_all_pairs_concurrent, measure_pair

    dev = dist_init("gloo" if a.internode else None)
    W, rank = dist.get_world_size(), dist.get_rank()
    res = {}
    if a.internode:
        per_node = int(os.environ.get("LOCAL_WORLD_SIZE", "1"))
        r = measure_pair(0, per_node if W > per_node else W - 1, a.send_msg_size, a.parallel, a.num_warmup, a.num_trials,
                         torch.device("cpu"))
        res = {"internode_bandwidth": r["bandwidth_gbs"], "internode_latency": r["latency_s"]}
    else:
        pairs = [(0, 1)] if (a.fast_intra or W < 3) else [(i, j) for i in range(W) for j in range(i + 1, W)]
        best = None
        for s, d in pairs:
            if W < 2:
                break
            r = measure_pair(s, d, a.send_msg_size, a.parallel, a.num_warmup, a.num_trials, dev)
            if best is None or r["bandwidth_gbs"] < best["bandwidth_gbs"]:
                best = r
        if best is None:
            best = {"bandwidth_gbs": 0.0, "latency_s": 0.0}
        res = {"intranode_bandwidth": best["bandwidth_gbs"], "intranode_latency": best["latency_s"]}
        if W >= 2:
            res["ring_shift_bandwidth_gbs"] = measure_all_pairs_concurrent(device=dev if dev.type == "cuda" else None,
                                                                           numel=16 * 1024 * 1024 if dev.type == "cuda" else 1 << 18)["bandwidth_gbs_per_direction"]
    if rank == 0:
        bw = res.get("intranode_bandwidth", res.get("internode_bandwidth", 0.0))
        lat = res.get("intranode_latency", res.get("internode_latency", 0.0))
        print(f"Bandwidth: {bw:.4f} GB/s")
        print(f"Latency: {lat:.6f} s")
        os.makedirs(a.output_dir, exist_ok=True)
        kind = "internode" if a.internode else "intranode"
        with open(os.path.join(a.output_dir, f"{kind}_bandwidth_results_{a.machine_index}.json"), "w") as f:
            json.dump(res, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
