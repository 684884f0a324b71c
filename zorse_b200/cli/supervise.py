"""Supervised training on one node: restart after a failure on the GPUs that are left.

    python -m zorse_b200.cli.supervise --config_file training_config.json --cluster_info_file cluster_info.json \
        --checkpoint_dir ck --train_steps 1000 --checkpoint_every 50 [--max_restarts 2] [--work_dir run] \
        -- [trainer flags, e.g. --one_f_one_b --heartbeat_timeout 120]

The supervisor starts one trainer process per rank of the plan (`zorse.py`, environment of a
torchrun job, rendezvous on 127.0.0.1) and waits.  A job that ends with every rank at exit code 0
is done.  Otherwise the ranks that failed are found from exit codes and logs: a rank that ended
with an error of its own (not the watchdog's abort code 3, not a signal from the supervisor, and a
log that does not read like the loss of a peer) is a failed rank; else the ranks the watchdog
reports name as not having entered the step the others are in (or as "behind or silent"); else
the rank that ended first.  The failed ranks' GPUs leave
the cluster description, the planner runs on what is left (`cli.recover`), and the job starts
again from the newest complete checkpoint under the new plan (with `--visible_devices`, every
process pinned to a surviving GPU).  The checkpoint reader re-shards across plans, and
`--train_steps` counts the steps of the checkpoint, so the restarted job trains the remaining
steps only.

There is no in-place resizing (a changed world is a new job), no multi-node launch (run one
supervisor per job on a node; across nodes the same steps apply with the site's launcher), and
no device-side fault detection beyond the trainer's own bounded waits and watchdog.  The reference
has neither checkpoints nor recovery.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import signal
import socket
import subprocess
import sys
import time
from typing import Optional

WATCHDOG_EXIT = 3          # cli/train.py: a rank whose watchdog saw no progress


def _free_port(also: int = 23) -> int:
    """A free rendezvous port whose `also`-th successor is free too (the trainer's heartbeat store listens there)."""
    for _ in range(50):
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        p = s.getsockname()[1]
        s.close()
        if p + also > 65535:
            continue
        t = socket.socket()
        try:
            t.bind(("127.0.0.1", p + also))
        except OSError:
            continue
        finally:
            t.close()
        return p
    raise RuntimeError("no pair of free ports found")


# what a rank prints when it fails because ANOTHER rank went away or fell silent
COLLATERAL = re.compile(r"Connection closed by peer|Connection reset|Broken pipe|Socket Timeout|Timed out waiting|"
                        r"NCCL|ncclRemoteError|ProcessGroup\w*[^\n]*(abort|timeout)|\[watchdog\]|recvBytes|sendBytes", re.I)


def failed_ranks(codes: dict, logs: dict, order: Optional[list] = None) -> list[int]:
    """Ranks to leave out of the next attempt.  `codes`: rank -> exit code (negative: ended by that signal).
    `logs`: rank -> what the rank printed.  `order`: ranks in the order in which they ended.

    1. ranks that ended with an error of their own: a non-zero code that is neither the watchdog's abort nor the
       supervisor's SIGTERM / SIGKILL, and a log that does not read like the loss of a peer;
    2. else the ranks the watchdog reports name as not having entered the step the others are in, else the ranks
       they name as behind or silent (a list that names every rank says nothing and is skipped);
    3. else the rank that ended first with an error."""
    errored = [r for r, c in codes.items()
               if c not in (0, None, WATCHDOG_EXIT) and not (c < 0 and -c in (signal.SIGTERM, signal.SIGKILL))]
    own = [r for r in errored if not COLLATERAL.search(logs.get(r) or "")]
    if own:
        return sorted(own)
    for pattern in (r"ranks that have not entered step \d+: \[([0-9, ]*)\]", r"ranks behind or silent: \[([0-9, ]*)\]"):
        named: set = set()
        for text in logs.values():
            for m in re.finditer(pattern, text or ""):
                named.update(int(x) for x in m.group(1).split(",") if x.strip())
        # a list that names every rank of the job says nothing (everybody waits behind the same step)
        if named and len(named) < len(codes):
            return sorted(named)
    for r in order or []:
        if r in errored:
            return [r]
    return sorted(errored)[:1]


def launch(world: int, trainer_argv: list[str], work_dir: str, attempt: int, devices: Optional[list[int]] = None,
           script: Optional[str] = None, poll_s: float = 0.02, grace_s: float = 30.0):
    """Runs one attempt; returns (codes, logs, ranks in the order they ended).  Once one rank has ended with an
    error the others get `grace_s` to end by themselves (their watchdogs name the silent ranks), then SIGTERM."""
    script = script or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "zorse.py")
    port = _free_port()
    procs, files = {}, {}
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), LOCAL_WORLD_SIZE=str(world),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        if devices is not None:
            env["CUDA_VISIBLE_DEVICES"] = str(devices[r])
            env["LOCAL_RANK"] = "0"
        path = os.path.join(work_dir, f"attempt{attempt}_rank{r}.log")
        files[r] = open(path, "w")
        procs[r] = subprocess.Popen([sys.executable, script] + trainer_argv, env=env, stdout=files[r], stderr=subprocess.STDOUT)
    first_error = None
    order: list = []
    while True:
        codes = {r: p.poll() for r, p in procs.items()}
        order += [r for r, c in codes.items() if c is not None and r not in order]
        if all(c is not None for c in codes.values()):
            break
        if first_error is None and any(c not in (None, 0) for c in codes.values()):
            first_error = time.time()
        if first_error is not None and time.time() - first_error > grace_s:
            for p in procs.values():
                if p.poll() is None:
                    p.terminate()
            deadline = time.time() + 10.0
            while time.time() < deadline and any(p.poll() is None for p in procs.values()):
                time.sleep(poll_s)
            for p in procs.values():
                if p.poll() is None:
                    p.kill()
        time.sleep(poll_s)
    codes = {r: p.wait() for r, p in procs.items()}
    logs = {}
    for r, f in files.items():
        f.close()
        with open(f.name) as g:
            logs[r] = g.read()
    return codes, logs, order


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    extra: list[str] = []
    if "--" in argv:
        i = argv.index("--")
        argv, extra = argv[:i], argv[i + 1:]
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config_file", required=True)
    ap.add_argument("--cluster_info_file", required=True, help="what the planner re-plans on after a failure")
    ap.add_argument("--checkpoint_dir", required=True)
    ap.add_argument("--train_steps", type=int, required=True)
    ap.add_argument("--checkpoint_every", type=int, default=10)
    ap.add_argument("--max_restarts", type=int, default=2)
    ap.add_argument("--work_dir", default="supervise_run", help="per-attempt configs and per-rank logs")
    ap.add_argument("--grace", type=float, default=30.0, help="seconds the other ranks get to end after the first error")
    ap.add_argument("--visible_devices", action="store_true",
                    help="pin every process to one GPU through CUDA_VISIBLE_DEVICES (surviving GPUs after a restart)")
    a = ap.parse_args(argv)
    from ..config.training_config import parse_pipeline_config
    from .recover import latest_checkpoint, replan, shrink_cluster

    os.makedirs(a.work_dir, exist_ok=True)
    with open(a.cluster_info_file) as f:
        cluster = json.load(f)
    alive = sorted(int(g["global_rank"]) for g in cluster["gpu_list"])       # original GPU numbers still in the job
    config = a.config_file
    for attempt in range(a.max_restarts + 1):
        cfg = parse_pipeline_config(config)
        world = cfg.world_size
        ck = latest_checkpoint(a.checkpoint_dir, verify=True)
        args = ["--config_file", config, "--checkpoint_dir", a.checkpoint_dir, "--checkpoint_every", str(a.checkpoint_every),
                "--train_steps", str(a.train_steps)] + (["--resume", ck] if ck else []) + extra
        if attempt > 0:
            args = [x for j, x in enumerate(args) if not (x == "--inject_fault" or (j > 0 and args[j - 1] == "--inject_fault"))]
        print(f"[supervise] attempt {attempt}: {world} ranks, config {config}, "
              f"{'from ' + ck if ck else 'from the start'}", flush=True)
        codes, logs, order = launch(world, args, a.work_dir, attempt, devices=alive[:world] if a.visible_devices else None,
                             grace_s=a.grace)
        if all(c == 0 for c in codes.values()):
            print(f"[supervise] done after {attempt} restart(s); newest checkpoint {latest_checkpoint(a.checkpoint_dir)}", flush=True)
            return 0
        bad = failed_ranks(codes, logs, order)
        print(f"[supervise] attempt {attempt} failed: exit codes {codes}; failed ranks {bad}", flush=True)
        if not bad or len(bad) >= world:
            print("[supervise] no rank can be singled out (see the per-rank logs); not restarting", flush=True)
            return 1
        if attempt == a.max_restarts:
            break
        ck = latest_checkpoint(a.checkpoint_dir, verify=True)
        # ranks of the failed attempt number the GPUs of the CURRENT cluster description
        cluster = shrink_cluster(cluster, bad)
        alive = [g for r, g in enumerate(alive) if r not in set(bad)]
        if ck is not None:
            from ..ckpt.reader import read_meta

            meta = read_meta(ck)
        else:
            with open(config) as f:
                meta = {"training_config": json.load(f)}
        new_cfg = replan(meta, cluster)
        config = os.path.join(a.work_dir, f"training_config_attempt{attempt + 1}.json")
        with open(config, "w") as f:
            json.dump(new_cfg, f, indent=1)
    print(f"[supervise] giving up after {a.max_restarts} restart(s)", flush=True)
    return 1


if __name__ == "__main__":
    raise SystemExit(main())
