#!/usr/bin/env python
"""Planner CLI:  python zorse_planner.py --cluster_info_file cluster_info.json --model_name ... --output plan.json

Flags follow the reference (zorse_planner.py:905-948; `--output` is accepted as a prefix of
`--output_file` there and explicitly here).
"""
import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cluster_info_file", required=True)
    ap.add_argument("--machine_file", default=None)
    ap.add_argument("--model_name", default="deepspeedllama_7b")
    ap.add_argument("--partition_algorithm", default="min_k_cut_split",
                    choices=["min_k_cut_split", "min_k_cut_efficient", "metis", "clustering"])
    ap.add_argument("--autocast_dtype", default="bfloat16")
    ap.add_argument("--reduce_dtype", default="float32")
    ap.add_argument("--num_trials", type=int, default=10)
    ap.add_argument("--num_warmup", type=int, default=3)
    ap.add_argument("--nccl_ib_disable", action="store_true")
    ap.add_argument("--vocab_size", type=int, default=32000)
    ap.add_argument("--dtype_multiplier", type=float, default=2.0)
    ap.add_argument("--optimizer_multiplier", type=float, default=12.0)
    ap.add_argument("--reserved_memory_gb", type=float, default=2.0)
    ap.add_argument("--global_batch_size", type=int, default=64)
    ap.add_argument("--sequence_length", type=int, default=4096)
    ap.add_argument("--output_file", "--output", dest="output_file", default="training_config.json")
    ap.add_argument("--use_agrs_comm_model", action="store_true",
                    help="cost all-gather / reduce-scatter with the model instead of profiling them")
    ap.add_argument("--agrs_profile", default=None, help="JSON of measured AG/RS times per group (profiler output)")
    ap.add_argument("--no_recompute", action="store_true")
    ap.add_argument("--num_stages", type=int, default=None, help="only try this number of GPU groups")
    ap.add_argument("--microbatch_size", type=int, default=None, help="plan for this microbatch size only (no sweep)")
    ap.add_argument("--tensor_parallel_size", type=int, default=1,
                    help="plan for lanes of this many GPUs that split every block (tensor parallelism); "
                         "the lane model is not calibrated against measurements yet")
    ap.add_argument("--compute_overhead", type=float, default=1.075,
                    help="whole-step time over the sum of profiled layer times (launch gaps, small kernels)")
    ap.add_argument("--graph_weighting", default="bandwidth", choices=["bandwidth", "mixed"],
                    help="edge weights of the GPU graph: link bandwidth alone, or mixed with memory and compute "
                         "similarity (keeps alike GPUs together where bandwidth ties; use with the clustering partitioner)")
    ap.add_argument("--schedule", default=None,
                    help="the schedule the trainer will run: candidate plans are ranked by this repository's prediction "
                         "for that schedule, and the file gets the schedule, that prediction and, with 1f1b, how many "
                         "of the last stage's layers hold their weight gradients back (defer_tail_wgrad)")
    ap.add_argument("--draw", default=None, help="write a PNG of the partitioned GPU graph (needs matplotlib)")
    a = ap.parse_args(argv)

    from zorse_b200.planner.cluster import load_cluster_info
    from zorse_b200.planner.plan import export_config, plan

    data = load_cluster_info(a.cluster_info_file)
    measured = None
    if a.agrs_profile and not a.use_agrs_comm_model:
        with open(a.agrs_profile) as f:
            measured = json.load(f)
    res, tried = plan(data, a.model_name, global_batch_size=a.global_batch_size, sequence_length=a.sequence_length,
                      autocast_dtype=a.autocast_dtype, reduce_dtype=a.reduce_dtype, vocab_size=a.vocab_size,
                      partition_algorithm=a.partition_algorithm, dtype_multiplier=a.dtype_multiplier,
                      optimizer_multiplier=a.optimizer_multiplier, reserved_memory_gb=a.reserved_memory_gb,
                      recompute=not a.no_recompute, measured_agrs=measured,
                      ks=[a.num_stages] if a.num_stages else None, microbatch_size=a.microbatch_size, compute_overhead=a.compute_overhead,
                      tensor_parallel_size=a.tensor_parallel_size, schedule=a.schedule,
                      graph_weighting=a.graph_weighting)
    for t in tried:
        print(f"k={t['k']}: predicted {t['latency_ms']} ms (microbatch {t['microbatch_size']}, interleave {t['interleave_degree']})"
              + (f"; under {a.schedule}: {t['schedule_ms']:.1f} ms" if t.get("schedule_ms") is not None else ""))
    if res is None:
        print("no plan fits in memory", file=sys.stderr)
        return 1
    cfg = export_config(res, a.model_name, a.global_batch_size, a.sequence_length, a.vocab_size, a.autocast_dtype,
                        a.reduce_dtype, a.output_file,
                        total_ranks=(int(data.get("total_gpus", 0)) // a.tensor_parallel_size) or None,
                        tensor_parallel_size=a.tensor_parallel_size)
    if a.schedule:
        from zorse_b200.planner.predict import best_tail_deferral, predict_step_ms

        cfg["schedule"] = a.schedule
        recompute = False if a.no_recompute else None
        try:
            if a.schedule == "1f1b" and a.tensor_parallel_size == 1 and res.interleave_degree == 1:
                cfg["defer_tail_wgrad"] = best_tail_deferral(cfg, a.schedule, recompute=recompute)
            cfg["latency"] = predict_step_ms(cfg, a.schedule, recompute=recompute,
                                             defer_tail_wgrad=cfg.get("defer_tail_wgrad", 0))["ms"]
            print(f"schedule {a.schedule}: predicted {cfg['latency']:.2f} ms"
                  + (f", defer_tail_wgrad {cfg['defer_tail_wgrad']}" if "defer_tail_wgrad" in cfg else ""))
        except Exception as e:      # noqa: BLE001 - no profile rows for this model on this GPU type
            print(f"schedule {a.schedule}: no prediction ({e!r}); the stage-2 estimate stays in the file", file=sys.stderr)
        with open(a.output_file, "w") as f:
            json.dump(cfg, f, indent=4)
    if cfg.get("unused_ranks"):
        print(f"ranks {cfg['unused_ranks']} own no stage (too slow to be given a layer); they idle during training")
    print(f"best: {len(res.stages)} stages, microbatch {res.microbatch_size}, interleave {res.interleave_degree}, "
          f"predicted {res.latency_ms:.2f} ms -> {a.output_file}")
    if a.draw:
        from zorse_b200.planner.partition import build_gpu_graph, partition
        from zorse_b200.planner.visualize import visualize_partition

        G = build_gpu_graph(data)
        visualize_partition(G, partition(G, len({tuple(s.gpu_ranks) for s in res.stages}), a.partition_algorithm), a.draw)
    return 0


if __name__ == "__main__":
    sys.exit(main())
