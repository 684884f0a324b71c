"""`zorse.py` main: parse flags + training config, build the job, run warm-up and measured
iterations, print the metrics block (reference zorse.py:109-283)."""
from __future__ import annotations

import os
import sys
import time

import torch
import torch.distributed as dist

from ..config.flags import parse_args_zorse
from ..config.training_config import parse_pipeline_config
from ..models import registry
from ..parallel import groups as G
from ..parallel.schedules import schedule_name_from_flags
from ..trainer import Trainer, TrainerOptions
from ..utils import metrics
from ..utils.logger import init_logger
from ..utils.pipeline_log import init_pipeline_logger


def main(argv=None) -> int:
    args = parse_args_zorse(argv)
    log = init_logger(args.log_level)
    cfg = parse_pipeline_config(args.config_file)
    if args.grad_norm_compat:
        cfg.grad_norm_compat = args.grad_norm_compat
    plog = init_pipeline_logger("./zorse_logs", int(os.environ.get("RANK", "0")), args.log_level) \
        if args.log_level == "DEBUG" else None
    opt = TrainerOptions(
        schedule=schedule_name_from_flags(args), ops=args.ops, optimizer_in_backward=args.optimizer_in_backwards,
        offload_model_params=args.offload_model_params, gloo_p2p=args.gloo_p2p, collectives=args.collectives,
        activation_recompute=False if args.no_recompute else None,
        activation_offload=True if args.offload_activations_to_host else None, lr=args.lr, seed=args.seed,
        backend=args.backend, pipeline_log=plog, shift_labels=args.shift_labels, defer_wgrad=args.defer_wgrad,
        defer_tail_wgrad=args.defer_tail_wgrad, prepost_recv=args.prepost_recv,
        p2p_timeout_s=args.p2p_timeout or None,
        p2p_fault_hooks=bool(args.inject_fault) and (":drop" in args.inject_fault or ":delay=" in args.inject_fault))
    if opt.defer_tail_wgrad < 0:
        # -1: the planner's rule decides (held-back work must fit into the time the other stages drain)
        opt.defer_tail_wgrad = 0
        if (cfg.schedule or opt.schedule) == "1f1b" and cfg.tensor_parallel_size == 1:
            try:
                from ..config.training_config import to_dict
                from ..planner.predict import best_tail_deferral

                opt.defer_tail_wgrad = best_tail_deferral(to_dict(cfg), "1f1b", recompute=opt.activation_recompute,
                                                          defer_wgrad=opt.defer_wgrad)
            except Exception as e:      # noqa: BLE001 - no profile table for this model / GPU: leave it off
                log.warning(f"--defer_tail_wgrad -1: no prediction for this model ({e!r}); off")
        log.info(f"defer_tail_wgrad = {opt.defer_tail_wgrad}")
    if args.nvtx:
        from ..utils import ranges

        ranges.enable()
    checker = None
    if args.check_streams and torch.cuda.is_available():
        from ..utils import stream_check

        checker = stream_check.install()
    if (len(cfg.stages) > 1 and torch.cuda.is_available() and args.backend != "gloo" and not opt.gloo_p2p
            and not args.no_preflight):
        # NCCL p2p between stages: replay the schedule's p2p program on the host first; a program that cannot
        # complete would leave the GPUs spinning in NCCL kernels until a timeout
        from ..parallel.p2p_sim import preflight

        name = cfg.schedule or opt.schedule
        stuck = None
        try:
            stuck = preflight(cfg, name, defer_wgrad=opt.defer_wgrad, prepost_recv=opt.prepost_recv)
        except Exception as e:      # noqa: BLE001 - the replay is a safety net, not a precondition
            log.warning(f"p2p replay skipped: {e!r}")
        if stuck is not None:
            raise SystemExit(f"schedule {name} would deadlock on this plan: {stuck} (try --gloo_p2p, --sync_comm or another schedule)")
    if args.inject_fault:
        from ..utils.health import injection_refusal

        refusal = injection_refusal(torch.cuda.is_available() and args.backend != "gloo", opt.collectives)
        if refusal:
            raise SystemExit(refusal)
    tr = Trainer(cfg, opt)
    resumed_step = 0
    log.info(f"rank {tr.rank}/{tr.world} on {tr.device}; schedule {tr.schedule.name}; ops {tr.ops.name}; "
             f"stages {[s.stage_id for s in tr.stages]}", leader_only=False)
    if args.resume:
        from ..ckpt.reader import load_checkpoint

        resumed_step = load_checkpoint(tr, args.resume)
        log.info(f"resumed from {args.resume} (step {resumed_step})")
    from ..utils.health import maybe_inject, parse_fault

    fault = parse_fault(args.inject_fault)
    watchdog = heartbeat = None
    if args.heartbeat_timeout > 0:
        import faulthandler

        from ..utils.health import Watchdog, tcp_heartbeat

        heartbeat = tcp_heartbeat(tr.rank, tr.world)
        entered = [None]          # the step this rank is in

        def stuck(step, idle):
            # name the ranks whose heartbeat is older than ours before giving up
            msg = f"[watchdog] rank {tr.rank}: no progress for {idle:.1f}s after step {step}"
            if heartbeat is not None:
                # half the limit: a peer that beat a moment after this rank's last beat is just as stuck
                behind = [r for r in heartbeat.stale_ranks(args.heartbeat_timeout / 2, min_step=step) if r != tr.rank]
                msg += f"; ranks behind or silent: {behind}"
                if entered[0] is not None:
                    # everybody who waits for a stuck rank looks "behind"; the rank that never started the step
                    # the others are in is the one they wait for
                    late = [r for r in heartbeat.not_entered(entered[0]) if r != tr.rank]
                    msg += f"; ranks that have not entered step {entered[0]}: {late}"
            sys.stderr.write(msg + "; dumping stacks and aborting\n")
            faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
            sys.stderr.flush()
            os._exit(3)

        watchdog = Watchdog(args.heartbeat_timeout, rank=tr.rank, on_timeout=stuck,
                            startup_s=args.heartbeat_startup or 10 * args.heartbeat_timeout)
        watchdog.start()
    batch = tr.synthetic_batch()
    inputs, targets, _ = tr.to_device(batch)
    cuda = tr.device.type == "cuda"
    if args.replay_check:
        from ..utils.replay import replay_check

        rep = replay_check(tr, inputs, targets)
        log.info(f"replay check: identical={rep['identical']} loss={rep['loss']} "
                 f"differing units={[(d['gid'], d['kind'], d['max_abs_diff']) for d in rep['differing_units']]}",
                 leader_only=False)
    # --train_steps: a job that is told how far to train and continues the count of the checkpoint it resumed;
    # otherwise the benchmark form of the reference (warm-up + timed iterations, counted from 0)
    first = resumed_step if args.train_steps else 0
    total = args.train_steps if args.train_steps else args.warmup_iterations + args.iterations
    if first >= total:
        log.info(f"checkpoint is at step {first}, --train_steps {total}: nothing left to train")
    iter_ms = []
    prof = None
    loss = None

    def report(avg_ms, loss):
        """The summary block (collective: every rank calls it): step time as the max over ranks, memory and GPU names
        over the host-side group, throughput, MFU, prediction, loss (reference utils/train_utils.py:556-734)."""
        t = torch.tensor([avg_ms, metrics.memory_stats(tr.device)["max_allocated_gb"]], dtype=torch.float64)
        gpu = metrics.clean_gpu_name(torch.cuda.get_device_name(tr.device)) if cuda else "cpu"
        if G.is_dist():
            grp = tr.gloo_group if tr.gloo_group is not None else None
            outs = [torch.zeros_like(t) for _ in range(tr.world)]
            names = [None] * tr.world
            if grp is not None or dist.get_backend() == "gloo":
                dist.all_gather(outs, t, group=grp)
                dist.all_gather_object(names, gpu, group=grp)
            else:
                outs, names = [t], [gpu]
        else:
            outs, names = [t], [gpu]
        step_ms = max(float(o[0]) for o in outs)
        spec = tr.spec
        flops = metrics.compute_model_flops(registry.total_params(spec, cfg.sequence_length), spec.layers, spec.hidden,
                                            cfg.sequence_length, cfg.global_batch_size, recompute=tr.schedule.recompute)
        gl = tr.global_loss(loss)
        predicted = cfg.latency
        if predicted is None and cuda:
            try:
                from ..config.training_config import to_dict
                from ..planner.predict import predict_step_ms

                # a job on several GPU models: every rank of the plan is costed with its own model's profile
                mixed = len(set(names)) > 1 and len(names) == tr.world and cfg.tensor_parallel_size == 1
                predicted = predict_step_ms(to_dict(cfg), tr.schedule.name, recompute=tr.schedule.recompute,
                                            gpu={i: n for i, n in enumerate(names)} if mixed else gpu,
                                            defer_wgrad=opt.defer_wgrad, defer_tail_wgrad=opt.defer_tail_wgrad)["ms"]
            except Exception:      # noqa: BLE001 - no profile table for this model / GPU: print no prediction
                predicted = None
        if tr.rank == 0:
            print(metrics.format_summary(global_batch=cfg.global_batch_size, seq=cfg.sequence_length, step_ms=step_ms,
                                         flops_per_step=flops, gpu_names=names, dtype=cfg.autocast_dtype,
                                         max_alloc_gb=[float(o[1]) for o in outs], predicted_ms=predicted, loss=gl,
                                         flashflex_ga=args.flashflex_ga), flush=True)

    for step in range(first, total):
        maybe_inject(fault, tr.rank, step, keepalive=watchdog.beat if watchdog else None,
                     transport=getattr(tr, "fault_transport", None))
        if heartbeat is not None:
            entered[0] = step
            heartbeat.beat_enter(step)
        if step - first == args.warmup_iterations:
            tr.synchronize()
            tr.barrier()
        if (not args.skip_profile and args.trace_dir and prof is None
                and step - first == args.warmup_iterations - args.profiling_iterations and args.profiling_iterations > 0):
            from ..utils.trace import profiler_context

            prof = profiler_context(args.trace_dir, args.experiment_name, tr.rank,
                                    unique_gpus_only=args.trace_unique_gpus_only)
            prof.__enter__()
        if cuda:
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record()
        ti = time.perf_counter()
        loss = tr.train_step(inputs, targets)
        if cuda:
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b)
        else:
            ms = (time.perf_counter() - ti) * 1e3
        tr.check_kernels()
        if watchdog:
            watchdog.beat(step)
        if heartbeat is not None:
            heartbeat.beat(step)
        if step - first == args.warmup_iterations - 3:
            # same point as the reference (zorse.py:170-172): three steps before the timed region
            metrics.print_memory_stats("before the timed steps", tr.device, rank=tr.rank,
                                       out=lambda line: log.info(line, leader_only=False))
        iter_ms.append(ms)
        log.info(f"Iteration {step} Time {ms:.2f} ms" + (f" loss {float(loss):.4f}" if loss is not None else ""))
        if prof is not None and step - first == args.warmup_iterations - 1:
            prof.__exit__(None, None, None)
            prof = None
        if args.print_metrics_every_iteration and args.warmup_iterations <= step - first < total - first - 1:
            # the running mean of the timed iterations so far, after each of them but the last (whose block is the
            # final one; reference zorse.py:185-196)
            so_far = iter_ms[args.warmup_iterations:]
            report(sum(so_far) / len(so_far), loss)
        if args.checkpoint_dir and args.checkpoint_every and (step + 1) % args.checkpoint_every == 0:
            from ..ckpt.writer import save_checkpoint

            save_checkpoint(tr, args.checkpoint_dir, step + 1)
    # mean of the timed iterations (each one is bracketed by events / a host clock and a device
    # synchronisation above), so checkpoint writes and logging between steps are not counted
    timed = iter_ms[args.warmup_iterations:] or iter_ms[-1:]
    avg_ms = sum(timed) / len(timed) if timed else 0.0
    tr.barrier()
    report(avg_ms, loss)
    if args.trace_dir and not args.skip_profile and args.profiling_iterations > 0:
        # stream-classified trace figures of this rank's profiled iterations (reference utils/train_utils.py:104-221,
        # printed from print_metrics when analyze_trace is set)
        from ..utils.trace import newest_trace, stream_overheads
        import os as _os

        tf = newest_trace(_os.path.join(_os.path.expanduser(args.trace_dir), args.experiment_name, f"GPU_{tr.rank}"))
        if tf:
            try:
                o = stream_overheads(tf, gap_threshold_us=args.gap_threshold)
                it = max(args.profiling_iterations, 1)
                log.info("trace: " + ", ".join(f"{k}={v / it:.2f}" for k, v in o.items() if isinstance(v, float))
                         + f" (ms per profiled iteration; streams {o['streams']})", leader_only=False)
            except (OSError, ValueError, KeyError) as e:
                log.warning(f"trace analysis skipped: {e!r}")
    if checker is not None:
        log.info(checker.report(), leader_only=False)
    if watchdog:
        watchdog.stop()
    if G.is_dist():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
