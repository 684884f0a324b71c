#!/usr/bin/env python
"""python collect_cluster_info.py --machine_file hostfile --output cluster_info.json

Lists the GPUs of every machine of the hostfile, measures intra- and inter-node bandwidth and
writes cluster_info.json for zorse_planner.py (reference collect_cluster_info.py:316-385)."""
import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--machine_file", default=None)
    ap.add_argument("--output", "--output_file", dest="output", default="cluster_info.json")
    ap.add_argument("--skip_bandwidth", action="store_true")
    ap.add_argument("--optimize_internode", action="store_true",
                    help="probe one representative machine pair per (region, GPU-set) class")
    ap.add_argument("--all_pairs_intra", action="store_true", help="probe every GPU pair instead of GPU 0 <-> 1")
    ap.add_argument("--fit_collectives", action="store_true", help="fit all-gather/reduce-scatter alpha and bandwidth")
    ap.add_argument("--fit_parameters", type=int, default=202383360)
    a = ap.parse_args(argv)
    from zorse_b200.profiler import cluster as C

    machines = C.read_machine_file(a.machine_file)
    info = C.collect_cluster_info(machines)
    if a.skip_bandwidth:
        info["bandwidth"] = {"internode_bandwidth": {}, "intranode_bandwidth": {str(i): 0.0 for i in range(len(machines))},
                             "internode_latency": {}, "intranode_latency": {str(i): 0.0 for i in range(len(machines))}}
    else:
        info["bandwidth"] = C.run_bandwidth_test(machines, info, optimize_internode=a.optimize_internode,
                                                 fast_intra=not a.all_pairs_intra)
    if a.fit_collectives and len(machines) == 1:
        info["collective_fit"] = C.fit_collectives_locally(info["machines"][0]["num_gpus"], a.fit_parameters)
    info["units"] = {"bandwidth": "GB/s", "latency": "seconds per probe message (10^7 float32 by default)",
                     "collective_fit": "alpha_ms in ms, bandwidth_gbs in GB/s per rank"}
    with open(a.output, "w") as f:
        json.dump(info, f, indent=4)
    print(f"wrote {a.output}: {info['total_gpus']} GPUs on {len(machines)} machine(s)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
