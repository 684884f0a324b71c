#!/usr/bin/env python
"""python comm_model.py --cluster_info_file cluster_info.json --model_name llama2_7b --ranks 0,1 [--dtype bfloat16]

Prints the modelled all-gather / reduce-scatter time of one layer's parameters over the given
ranks (reference comm_model.py:116-162)."""
import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cluster_info_file", required=True)
    ap.add_argument("--model_name", default="llama2_7b")
    ap.add_argument("--ranks", default=None, help="comma separated global ranks (default: all)")
    ap.add_argument("--dtype", default="bfloat16")
    a = ap.parse_args(argv)
    from zorse_b200.models import registry
    from zorse_b200.planner import comm_model as cm
    from zorse_b200.planner.cluster import load_cluster_info

    data = load_cluster_info(a.cluster_info_file)
    ranks = [int(r) for r in a.ranks.split(",")] if a.ranks else [g["global_rank"] for g in data["gpu_list"]]
    P = registry.get_model_stats(a.model_name)["parameters_per_layer"]
    size = cm.tensor_size_bytes(P, a.dtype)
    bw = cm.bandwidth_matrix(data, ranks)
    print(f"tensor: {P} parameters, {size / 1e9:.4f} GB ({a.dtype})")
    print(f"ring (slowest link):        {cm.ring_collective_ms(size, bw):.3f} ms")
    print(f"ring v2 (per-step, x1.15):  {cm.ring_collective_ms_v2(size, bw):.3f} ms")
    print(f"all_gather (best model):    {cm.collective_ms(data, ranks, size, 'all_gather'):.3f} ms")
    print(f"reduce_scatter (best model): {cm.collective_ms(data, ranks, size, 'reduce_scatter'):.3f} ms")
    return 0


if __name__ == "__main__":
    sys.exit(main())
