"""Runs the unmodified reference trainer (the copy of its tree under `baseline/_ref/`) on the
benchmark configuration and times it the way `bench.py` times this repository's own arm.

The reference is started through its own entry point (`zorse.py:main`, reference `zorse.py:212-283`)
with its own flags and a `training_config.json` written for the run; its schedules, its patched
FSDP engine, its models and its optimizer run as shipped.  Nothing of this repository's package
is imported.  What this harness adds around it, without editing a reference file:

* `ref_shim.install()` before the reference's modules are imported (names that the installed
  transformers release removed) and `ref_shim.patch_tables()` after (B200 / bf16 table rows);
* a wrapper around the schedule's `step` that places barrier + synchronize + CUDA-event marks at
  the boundaries of the timed regions (the reference prints per-rank times on local rank 0 only,
  reference `zorse.py:183-201`; the benchmark wants the maximum over ranks);
* a second timed region in which every step first copies its token ids and labels from pinned
  host memory into the reference's device tensors and afterwards reads the last loss back
  (the reference creates its inputs once on the device, `zorse.py:41-47,73-85`, and never reads a loss).

A failure anywhere prints one `{"impl": "reference", "unavailable": ...}` line and every rank exits 0.
"""
from __future__ import annotations

import json
import os
import sys
import tempfile
import threading
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")

REF_MODEL = {"llama2_7b": "deepspeedllama_7b", "llama_tiny": "deepspeedllama_tiny", "llama2_13b": "deepspeedllama_13b"}
SCHEDULE_FLAG = {"zero2": "--zero2_pipeline", "layer_major": None, "no_overlap": "--sync_comm",
                 "two_stage_sync": "--two_stage_sync", "flashflex": "--flashflex_pipeline"}


def stage_plan(n: int, layers: int):
    """Same rank groups and layer ranges per N as the repository's own arm."""
    if n == 1:
        return [([0], 0, layers)], "pp1xdp1"
    if n == 2:
        return [([0, 1], 0, layers)], "pp1xdp2-zero3"
    if n == 4:
        h = layers // 2
        return [([0, 1], 0, h), ([2, 3], h, layers)], "pp2xdp2-zero3"
    if n == 8:
        q = layers // 4
        return [([2 * i, 2 * i + 1], i * q, (i + 1) * q if i < 3 else layers) for i in range(4)], "pp4xdp2-zero3"
    raise SystemExit(f"1, 2, 4 or 8 GPUs, got {n}")


def write_config(path, n, model, layers, gbs, mbs, seq, vocab, reduce_dtype):
    stages, par = stage_plan(n, layers)
    M = gbs // mbs
    pipe = []
    for ranks, a, b in stages:
        base, rem = divmod(M, len(ranks))
        pipe.append({"gpu_ranks": ranks, "layer_partition": [a, b], "zero_config": [ranks],
                     "num_microbatches_per_rank": [base + (1 if i < rem else 0) for i in range(len(ranks))]})
    cfg = {"model_name": model, "global_batch_size": gbs, "microbatch_size": mbs, "sequence_length": seq,
           "vocab_size": vocab, "fused_optimizer": True, "autocast_dtype": "bfloat16", "reduce_dtype": reduce_dtype,
           "split_microbatches_evenly": True, "pipeline_config": pipe}
    with open(path, "w") as f:
        json.dump(cfg, f)
    return par


class _Abort:
    """One rank's failure ends every rank with exit code 0 (a marker file in the run's scratch
    directory, polled by a thread on each rank), so the job never sits in a collective that a
    dead peer cannot join."""

    def __init__(self, scratch, rank):
        self.marker, self.rank = os.path.join(scratch, "ABORT"), rank
        self.stop = threading.Event()
        self.last_progress = time.time()
        threading.Thread(target=self._poll, daemon=True).start()

    def _poll(self):
        while not self.stop.wait(0.5):
            if os.path.exists(self.marker):
                os._exit(0)

    def fail(self, why: str):
        first = False
        try:
            fd = os.open(self.marker, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
            os.write(fd, why.encode()[:2000])
            os.close(fd)
            first = True
        except FileExistsError:
            pass
        if first:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        time.sleep(1.5)
        os._exit(0)


def one_line(exc: BaseException) -> str:
    tb = traceback.extract_tb(exc.__traceback__)
    where = ""
    for fr in reversed(tb):
        if "_ref" in fr.filename or "torch/distributed/fsdp" in fr.filename:
            where = f" at {os.path.relpath(fr.filename, REF_ROOT) if '_ref' in fr.filename else fr.filename.split('site-packages/')[-1]}:{fr.lineno}"
            break
    msg = " ".join(str(exc).split())
    return f"reference run failed on this box: {type(exc).__name__}: {msg[:400]}{where}"


def run(args, clock_sampler_cls=None) -> int:
    n, K, W = args.gpus, args.steps, max(3, args.warmup)
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_WORLD_SIZE", os.environ["WORLD_SIZE"])
    os.environ.setdefault("GROUP_RANK", "0")
    os.environ.setdefault("GROUP_WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if world != n:
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}; launch with torch.distributed.run for N > 1")
    if not os.path.isdir(os.path.join(REF_ROOT, "zorse_utils")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref does not hold the reference tree"}))
        return 0
    scratch = os.path.join(tempfile.gettempdir(), f"zorse_ref_{os.environ['MASTER_PORT']}_{os.getppid() if world > 1 else os.getpid()}")
    os.makedirs(scratch, exist_ok=True)
    abort = _Abort(scratch, rank)
    try:
        return _run(args, n, K, W, rank, world, scratch, abort, clock_sampler_cls)
    except SystemExit:
        raise
    except BaseException as e:      # noqa: BLE001 - every failure becomes the one-line record
        sys.stderr.write(traceback.format_exc())
        abort.fail(one_line(e))
    return 0


def _run(args, n, K, W, rank, world, scratch, abort, clock_sampler_cls) -> int:
    sys.path.insert(0, HERE)
    sys.path.insert(0, REF_ROOT)
    import ref_shim

    added = ref_shim.install()
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    if not torch.cuda.is_available():
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device: the reference engine is FSDP on CUDA streams"}))
        return 0

    model = REF_MODEL.get(args.model, args.model)
    os.chdir(scratch)                      # the reference writes ./zorse_logs relative to the working directory
    import zorse as ref                    # the reference's entry module
    from models.hub import get_config_for_model

    ref_shim.patch_tables()
    layers = args.layers or get_config_for_model(model)[0]
    cfg_path = os.path.join(scratch, f"training_config_rank{rank}.json")
    par = write_config(cfg_path, n, model, layers, args.global_batch, args.microbatch, args.seq_len, args.vocab,
                       args.reduce_dtype)
    sched = getattr(args, "ref_schedule", "zero2")
    do_e2e = not args.skip_e2e
    argv = ["zorse.py", "--config_file", cfg_path, "--model_name", model, "--iterations", str(K * (2 if do_e2e else 1)),
            "--warmup_iterations", str(W), "--skip_profile", "--trace_dir", os.path.join(scratch, "traces"),
            "--log_level", "WARNING"]
    if SCHEDULE_FLAG[sched]:
        argv.append(SCHEDULE_FLAG[sched])
    if args.optimizer_in_backward:
        argv.append("--optimizer_in_backwards")
    sys.argv = argv

    st = {"ev": {}, "wall": {}, "loss": None, "host_in": None, "host_tg": None, "h2d": 0, "d2h": 0, "steps_done": 0,
          "sampler": None}

    real_ce = F.cross_entropy

    def ce(*a, **k):
        out = real_ce(*a, **k)
        st["loss"] = out.detach()
        return out

    F.cross_entropy = ce
    torch.nn.functional.cross_entropy = ce

    def mark(name):
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        st["ev"][name] = e
        st["wall"][name] = time.perf_counter()

    def wrap_schedule(build):
        def build_wrapped(*a, **k):
            sch = build(*a, **k)
            real_step = sch.step

            def step(step_idx, input_chunks=None, target_chunks=None):
                if step_idx == W:
                    if rank == 0 and clock_sampler_cls is not None:
                        st["sampler"] = clock_sampler_cls(int(os.environ.get("LOCAL_RANK", "0")))
                        st["sampler"].start()
                    mark("t0")
                if step_idx == W + K:
                    mark("t1")
                    if do_e2e:
                        st["host_in"] = [c.cpu().pin_memory() for c in (input_chunks or [])]
                        st["host_tg"] = [c.cpu().pin_memory() for c in (target_chunks or [])]
                        mark("e0")
                e2e_step = do_e2e and step_idx >= W + K
                if e2e_step:
                    for dev, host in zip(input_chunks or [], st["host_in"]):
                        dev.copy_(host, non_blocking=True)
                        st["h2d"] += host.numel() * host.element_size()
                    for dev, host in zip(target_chunks or [], st["host_tg"]):
                        dev.copy_(host, non_blocking=True)
                        st["h2d"] += host.numel() * host.element_size()
                out = real_step(step_idx, input_chunks=input_chunks, target_chunks=target_chunks)
                if e2e_step and target_chunks and st["loss"] is not None:
                    st["loss_value"] = float(st["loss"].float().item())
                    st["d2h"] += 4
                st["steps_done"] += 1
                abort.last_progress = time.time()
                return out

            sch.step = step
            return sch

        return build_wrapped

    for name in ("build_pipeline_schedule", "build_pipeline_schedule_sync", "build_pipeline_schedule_two_stage_sync",
                 "build_pipeline_schedule_zero2", "build_pipeline_schedule_flashflex"):
        setattr(ref, name, wrap_schedule(getattr(ref, name)))

    real_print_metrics = ref.print_metrics
    result = {}

    def print_metrics(*a, **k):
        # called once after the reference's loop (reference zorse.py:198-209): close the last region here
        if "done" in result:
            return
        mark("t2")
        tokens = args.global_batch * args.seq_len
        ms = st["ev"]["t0"].elapsed_time(st["ev"]["t1"] if "t1" in st["ev"] else st["ev"]["t2"]) / K
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        result.update(done=True, ms=float(t.item()), tokens=tokens)
        if do_e2e:
            wall = (st["wall"]["t2"] - st["wall"]["e0"]) / K * 1e3
            w = torch.tensor([wall], device="cuda")
            dist.all_reduce(w, op=dist.ReduceOp.MAX)
            b = torch.tensor([float(st["h2d"]) / K, float(st["d2h"]) / K], device="cuda")
            dist.all_reduce(b)
            result.update(e2e_ms=float(w.item()), h2d=int(b[0].item()), d2h=int(b[1].item()))
        try:
            real_print_metrics(*a, **k)
        except Exception as e:      # noqa: BLE001 - the reference's summary printer is not part of the measurement
            sys.stderr.write(f"[ref_harness] reference print_metrics raised {e!r}\n")

    ref.print_metrics = print_metrics

    stall = float(getattr(args, "stall_timeout", 900.0)) * 2

    def stall_watch():
        while not abort.stop.wait(5.0):
            if time.time() - abort.last_progress > stall:
                abort.fail(f"reference run stalled: no step finished for {stall:.0f}s after step {st['steps_done']}")

    threading.Thread(target=stall_watch, daemon=True).start()

    ref.main()

    abort.stop.set()
    if rank == 0:
        sampler = st["sampler"]
        clocks = None
        if sampler is not None:
            sampler.stop_flag.set()
            sampler.join(timeout=2)
            clocks = sampler.summary()
        value = result["tokens"] / (result["ms"] / 1e3)
        out = {"metric": "tokens/s", "value": value, "unit": "tokens/s", "n_gpus": n, "steps": K, "warmup": W,
               "ms_per_step": result["ms"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
               "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights", "impl": "reference",
               "config": {"model": args.model + ("" if args.layers is None else f"[layers={args.layers} DEBUG]"),
                          "global_batch": args.global_batch, "seq_len": args.seq_len, "microbatch": args.microbatch,
                          "parallelism": par, "schedule": sched + " (reference flag " + str(SCHEDULE_FLAG[sched]) + ")",
                          "activation_recompute": True,
                          "optimizer": "torch.optim.Adam(fused) on fp32 FSDP flat parameters, step inside the timed region",
                          "reduce_dtype": args.reduce_dtype, "collectives": "NCCL through the reference's patched FSDP",
                          "reference_model": model, "shim": added,
                          "l2": "per-step working set far exceeds the 126 MB L2; no flush needed"},
               "clocks": clocks, "gpu_launches": 0, "loss": st.get("loss_value"),
               "max_memory_allocated_gb_rank0": torch.cuda.max_memory_allocated() / 2**30}
        if do_e2e:
            out["e2e"] = {"value": result["tokens"] / (result["e2e_ms"] / 1e3), "unit": "tokens/s",
                          "ms_per_step": result["e2e_ms"], "h2d_bytes_per_step": result["h2d"],
                          "d2h_bytes_per_step": result["d2h"]}
        print(json.dumps(out), flush=True)
    return 0
