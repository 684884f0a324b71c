"""Command-line flags of the trainer.

The flags that change behaviour are the ones the reference trainer reads
(zorse_utils/argparse.py:37-215, zorse.py:212-283): `--config_file`, the schedule selectors,
`--gloo_p2p`, `--offload_model_params`, `--optimizer_in_backwards`, iteration counts,
profiling and logging options.  The reference parses some fifty more flags inherited from
an older trainer and ignores them; they are accepted here as well (with a warning) so
existing command lines keep working.  Every top-level key of the training-config JSON
overrides the attribute of the same name (dtype strings become torch dtypes and
`sequence_length` becomes `seq_length`), as `override_args_with_config` does (:25-34).
"""
from __future__ import annotations

import argparse
import json
import warnings

from .training_config import dtype_from_str

# flags the reference accepts but its pipeline trainer never reads: (name, takes a value)
_IGNORED = [
    ("model_name", True), ("cluster", True), ("vocab_size", True), ("batch_size", True), ("microbatches", True),
    ("seq_length", True), ("image_size", True), ("full_shard_layers", True), ("recompute_layers", True),
    ("no_fused_optimizer", False), ("recompute_layer", False), ("recompute_feed_forward", False),
    ("recompute_attention", False), ("cpu_offload", False), ("offload_activations", False),
    ("sync_backwards", False), ("compile", False), ("no_shard", False), ("hybrid_shard", False),
    ("hybrid_shard_groups", True), ("reverse_hs", False), ("split_uneven", False), ("ga", True),
    ("proportional_split", False), ("profile_memory", False), ("profile_ga", False),
    ("use_activation_buffers", False), ("detailed_profiler_trace", False), ("use_prefetch_backwards", False),
    ("use_forwards_gpu_buffer", False), ("unshard_in_compute", False), ("async_tp", False),
    ("enable_loss_parallel", False), ("compile_transformer_blocks", False), ("split_uneven_partitions", True),
    ("uneven_batch_sizes", True), ("uneven_microbatches", True), ("scale_config_bs", True), ("tt_pp", True),
    ("zero2", False), ("tt_pp_schedule", True), ("tt_dp_shard", True), ("tt_dp_replicate", True), ("tt_tp", True),
    ("tt_pp_split_points", True), ("tt_pp_microbatches", True), ("use_deepcopy_for_build", False), ("mfu_gpus", True),
]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="zorse-b200 pipeline + ZeRO trainer")
    p.add_argument("--config_file", type=str, required=True, help="training_config.json written by the planner")
    p.add_argument("--log_level", default="INFO", choices=["DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"])
    p.add_argument("--autocast_dtype", default="bfloat16")
    p.add_argument("--reduce_dtype", default="float32")
    p.add_argument("--iterations", type=int, default=4)
    p.add_argument("--warmup_iterations", type=int, default=5)
    p.add_argument("--profiling_iterations", type=int, default=2)
    p.add_argument("--skip_profile", action="store_true")
    p.add_argument("--trace_dir", type=str, default=None)
    p.add_argument("--experiment_name", type=str, default="zorse")
    p.add_argument("--gap_threshold", type=float, default=0.0)
    p.add_argument("--optimizer_in_backwards", action="store_true")
    p.add_argument("--sync_comm", action="store_true", help="no-overlap schedule")
    p.add_argument("--two_stage_sync", action="store_true")
    p.add_argument("--zero2_pipeline", action="store_true")
    p.add_argument("--flashflex_pipeline", action="store_true")
    p.add_argument("--flashflex_ga", type=int, default=1)
    p.add_argument("--gloo_p2p", action="store_true")
    p.add_argument("--offload_model_params", action="store_true")
    p.add_argument("--print_metrics_every_iteration", action="store_true")
    # additions of this framework
    p.add_argument("--one_f_one_b", action="store_true", help="true 1F1B schedule")
    p.add_argument("--schedule", default=None, help="explicit schedule name (overrides the selector flags)")
    p.add_argument("--ops", default=None, choices=["sm100", "ref"], help="kernel backend (default: sm100 on CUDA)")
    p.add_argument("--collectives", default="library", choices=["library", "fused"],
                   help="ZeRO collectives: NCCL/gloo calls, or in-kernel NVLink kernels fused with Adam / GEMM")
    p.add_argument("--backend", default=None, choices=["nccl", "gloo"])
    p.add_argument("--grad_norm_compat", default=None, choices=["mean", "reference"])
    p.add_argument("--no_recompute", action="store_true", help="keep activations instead of recomputing layers")
    p.add_argument("--offload_activations_to_host", action="store_true")
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--checkpoint_dir", type=str, default=None)
    p.add_argument("--checkpoint_every", type=int, default=0)
    p.add_argument("--resume", type=str, default=None)
    p.add_argument("--trace_unique_gpus_only", action="store_true",
                   help="profiler traces only on the first GPU of each model per machine (the reference's behaviour); "
                        "default: every rank records its own")
    p.add_argument("--p2p_timeout", type=float, default=0.0,
                   help="Gloo p2p: seconds a pipeline receive may wait before the job fails with the name of the missing "
                        "message (0: the process group's timeout)")
    p.add_argument("--train_steps", type=int, default=0,
                   help="train up to this optimizer step, counting the steps of a resumed checkpoint (checkpoints and "
                        "--inject_fault then use that global step); 0 = run --warmup_iterations + --iterations steps")
    p.add_argument("--no_preflight", action="store_true",
                   help="skip the host-side replay of the schedule's p2p program before a multi-stage NCCL job starts")
    p.add_argument("--prepost_recv", action="store_true",
                   help="1F1B: post the receive of the next forward / backward before computing the current one "
                        "(stage boundaries then use their own process groups); not measured on hardware")
    p.add_argument("--defer_tail_wgrad", type=int, default=0,
                   help="1F1B: weight gradients of the last stage's last N layers (the output head first) run after the "
                        "stage's last backward, in the time it otherwise idles while the other stages drain "
                        "(-1: the planner's rule picks N for the plan)")
    p.add_argument("--defer_wgrad", action="store_true",
                   help="1F1B schedules: send each microbatch's input gradient upstream before its weight-gradient GEMMs run")
    p.add_argument("--heartbeat_timeout", type=float, default=0.0, help="seconds; 0 disables the watchdog")
    p.add_argument("--heartbeat_startup", type=float, default=0.0,
                   help="seconds the first step may take (default: ten times --heartbeat_timeout)")
    p.add_argument("--inject_fault", type=str, default=None,
                   help="testing: rank:step:kind (stall | raise | exit), a host-side failure of one rank between steps")
    p.add_argument("--shift_labels", action="store_true",
                   help="targets = next token of the inputs (last position ignored) instead of random targets")
    p.add_argument("--nvtx", action="store_true", help="name every engine phase (NVTX + profiler record_function)")
    p.add_argument("--check_streams", action="store_true",
                   help="debug: host-side check that every buffer read was ordered after its last write")
    p.add_argument("--replay_check", action="store_true",
                   help="debug: run the first step twice from the same state and compare the results bit by bit")
    for name, has_val in _IGNORED:
        if has_val:
            p.add_argument(f"--{name}", default=None, help=argparse.SUPPRESS)
        else:
            p.add_argument(f"--{name}", action="store_true", help=argparse.SUPPRESS)
    return p


def override_args_with_config(args) -> None:
    with open(args.config_file) as f:
        cfg = json.load(f)
    for k, v in cfg.items():
        if k == "pipeline_config":
            continue
        if k in ("autocast_dtype", "reduce_dtype"):
            v = dtype_from_str(v)
        if k == "sequence_length":
            k = "seq_length"
        setattr(args, k, v)


def parse_args_zorse(argv=None):
    p = build_parser()
    args = p.parse_args(argv)
    used = [n for n, has_val in _IGNORED
            if (getattr(args, n) is not None if has_val else getattr(args, n))]
    if used:
        warnings.warn("flags accepted for compatibility and ignored: " + ", ".join("--" + n for n in used))
    override_args_with_config(args)
    return args
