"""Checkpoint round trip / re-sharding and host-side failure detection (no GPU involved)."""
import os
import time

import pytest
import torch

from dist_utils import run_workers
from zorse_b200.config.training_config import parse_pipeline_dict
from zorse_b200.utils.health import DictStore, Heartbeat, Watchdog
from test_dist_cpu import PIPE_1x2, PIPE_2x1, tiny_cfg


def _train_and_save(rank, world, cfg_dict, ckdir, steps):
    from zorse_b200.ckpt.writer import save_checkpoint
    from zorse_b200.trainer import Trainer, TrainerOptions

    tr = Trainer(parse_pipeline_dict(cfg_dict), TrainerOptions(backend="gloo", schedule="layer_major"))
    batch = tr.synthetic_batch()
    for _ in range(steps):
        tr.train_step_from_host(batch)
    save_checkpoint(tr, ckdir, steps)
    return tr.global_loss(tr.train_step_from_host(batch))


def _load_and_step(rank, world, cfg_dict, ckdir, steps):
    from zorse_b200.ckpt.reader import load_checkpoint
    from zorse_b200.trainer import Trainer, TrainerOptions

    tr = Trainer(parse_pipeline_dict(cfg_dict), TrainerOptions(backend="gloo", schedule="layer_major", seed=0))
    assert load_checkpoint(tr, os.path.join(ckdir, f"step_{steps}")) == steps
    batch = tr.synthetic_batch()
    return tr.global_loss(tr.train_step_from_host(batch))


def test_checkpoint_resume_and_reshard(tmp_path):
    ck = str(tmp_path / "ck")
    a = run_workers(2, _train_and_save, tiny_cfg(PIPE_2x1), ck, 2)
    # same plan
    b = run_workers(2, _load_and_step, tiny_cfg(PIPE_2x1), ck, 2)
    assert abs(a[0] - b[0]) < 1e-5, (a, b)
    # different plan: one stage, 2-way sharded
    c = run_workers(2, _load_and_step, tiny_cfg(PIPE_1x2), ck, 2)
    assert abs(a[0] - c[0]) < 1e-4, (a, c)


def test_checkpoint_reshard_from_unequal_shards(tmp_path):
    ck = str(tmp_path / "ck")
    uneven = [dict(PIPE_1x2[0], shard_ratio=[3, 1])]
    a = run_workers(2, _train_and_save, tiny_cfg(uneven), ck, 2)
    b = run_workers(2, _load_and_step, tiny_cfg(PIPE_1x2), ck, 2)       # -> equal shards
    assert abs(a[0] - b[0]) < 1e-4, (a, b)
    d = run_workers(2, _load_and_step, tiny_cfg([dict(PIPE_1x2[0], shard_ratio=[1, 2])]), ck, 2)
    assert abs(a[0] - d[0]) < 1e-4, (a, d)


def test_corrupt_checkpoint_is_detected(tmp_path):
    from zorse_b200.ckpt.reader import CheckpointError, read_meta

    ck = str(tmp_path / "ck")
    run_workers(2, _train_and_save, tiny_cfg(PIPE_2x1), ck, 1)
    d = os.path.join(ck, "step_1")
    f = os.path.join(d, "stage0_rank0.bin")
    with open(f, "r+b") as fh:
        fh.truncate(os.path.getsize(f) // 2)
    with pytest.raises(RuntimeError, match="truncated"):
        run_workers(2, _load_and_step, tiny_cfg(PIPE_2x1), ck, 1, timeout=120)
    import numpy as np

    from zorse_b200.ckpt.reader import main as verify_main, verify_checkpoint

    with pytest.raises(CheckpointError, match="truncated"):
        verify_checkpoint(d)
    assert verify_main([d]) == 2
    os.remove(os.path.join(d, "meta.json"))
    with pytest.raises(CheckpointError):
        read_meta(d)
    # an intact checkpoint verifies; a NaN written into a shard file is found and located
    ck2 = str(tmp_path / "ck2")
    run_workers(2, _train_and_save, tiny_cfg(PIPE_2x1), ck2, 1)
    d2 = os.path.join(ck2, "step_1")
    ok = verify_checkpoint(d2)
    assert ok["step"] == 1 and ok["files"] == 2 and not ok["bad_units"] and ok["model"] == "tiny_llama"
    assert verify_main([d2]) == 0
    with open(os.path.join(d2, "stage1_rank1.bin"), "r+b") as fh:
        fh.seek(8)
        fh.write(np.array([np.nan], dtype="<f4").tobytes())
    bad = verify_checkpoint(d2)
    assert len(bad["bad_units"]) == 1 and bad["bad_units"][0][0] == 1 and bad["bad_units"][0][3] == "master"
    assert verify_main([d2]) == 1 and verify_main([d2, "--no-values"]) == 0


def test_heartbeat_names_the_silent_rank():
    now = [1000.0]
    store = DictStore()
    hbs = [Heartbeat(store, r, 3, clock=lambda: now[0]) for r in range(3)]
    for h in hbs:
        h.beat(0)
    now[0] += 5
    hbs[0].beat(1)
    hbs[2].beat(1)       # rank 1 never reports step 1
    now[0] += 5
    assert hbs[0].stale_ranks(limit_s=8.0) == [1]
    assert hbs[0].stale_ranks(limit_s=100.0, min_step=1) == [1]
    # ranks 0 and 2 wait inside step 2 for rank 1, which never started it: all three have finished step 1 at best,
    # but only rank 1 has not entered step 2
    hbs[1].beat(1)
    for r in (0, 1, 2):
        hbs[r].beat_enter(1)
    hbs[0].beat_enter(2)
    hbs[2].beat_enter(2)
    assert hbs[0].not_entered(2) == [1] and hbs[0].not_entered(1) == [] and hbs[0].not_entered(3) == [0, 1, 2]


def test_short_or_garbled_store_reads_count_as_silence():
    """A store that returns a cut-off or mangled heartbeat value (short read) or raises: the rank is reported as
    silent; the reader does not crash the watchdog that calls it."""
    class BadStore(DictStore):
        def __init__(self, bad):
            super().__init__()
            self.bad = bad

        def get(self, k):
            if k in self.bad:
                v = self.bad[k]
                if isinstance(v, Exception):
                    raise v
                return v
            return super().get(k)

    now = [50.0]
    store = BadStore({"hb/1": b"12", "hb/2": "7:", "hb/3": "x:y", "hb/4": RuntimeError("store gone"), "hb/5": b""})
    hbs = [Heartbeat(store, r, 6, clock=lambda: now[0]) for r in range(6)]
    for h in hbs:
        h.beat(3)
    assert hbs[0].read(0) == (3, 50.0) and all(hbs[0].read(r) is None for r in range(1, 6))
    assert hbs[0].stale_ranks(limit_s=10.0) == [1, 2, 3, 4, 5]


def test_watchdog_fires_on_a_stuck_step():
    fired = []
    w = Watchdog(1.0, on_timeout=lambda step, idle: fired.append((step, idle)), poll_s=0.05)
    w.start()
    w.beat(7)
    time.sleep(0.2)
    w.beat(8)
    time.sleep(0.2)
    assert not fired
    time.sleep(1.3)
    assert fired and fired[0][0] == 8
    w.stop()


def test_watchdog_allows_a_slow_first_step():
    """Until the first beat the longer start-up limit applies; afterwards the normal one."""
    fired = []
    w = Watchdog(0.2, on_timeout=lambda step, idle: fired.append((step, idle)), poll_s=0.05, startup_s=1.0)
    w.start()
    time.sleep(0.5)
    assert not fired            # 0.5 s without any beat: inside the start-up limit
    w.beat(0)
    time.sleep(0.5)
    assert fired and fired[0][0] == 0
    w.stop()
    fired2 = []
    w2 = Watchdog(0.2, on_timeout=lambda step, idle: fired2.append(step), poll_s=0.05, startup_s=0.4)
    w2.start()
    time.sleep(0.8)
    assert fired2 == [-1]       # a first step that never ends is still caught
    w2.stop()


def _rank_that_dies(rank, world):
    """A rank that raises before joining a collective: the others see a bounded failure."""
    import datetime

    import torch.distributed as dist

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        raise RuntimeError("injected host-side fault")
    t = torch.ones(1)
    try:
        dist.all_reduce(t)
    except Exception as e:  # the surviving rank gets an error, not a hang
        return f"error: {type(e).__name__}"
    return "no error"


def test_peer_failure_ends_collective_with_error():
    with pytest.raises(RuntimeError, match="injected host-side fault|rank 0 failed|exited"):
        run_workers(2, _rank_that_dies, timeout=90)


def test_cli_watchdog_names_the_rank_that_stopped(tmp_path):
    """Two gloo ranks under torchrun; rank 1 stops joining before step 2 (host-side fault
    injection). Rank 0's next receive never completes, its watchdog fires, reads the heartbeat
    store and names rank 1 before aborting."""
    import json
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(tiny_cfg(PIPE_2x1, fused_optimizer=True)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29911", os.path.join(root, "zorse.py"), "--config_file", str(cfg_file),
           "--backend", "gloo", "--ops", "ref", "--iterations", "3", "--warmup_iterations", "3", "--skip_profile",
           "--heartbeat_timeout", "6", "--inject_fault", "1:2:stall"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=dict(os.environ, PYTHONPATH=root), cwd=root)
    out = r.stdout + r.stderr
    assert r.returncode != 0
    assert "[watchdog] rank 0: no progress" in out, out[-3000:]
    assert "ranks behind or silent: [1]" in out, out[-3000:]


def test_read_range_against_synthetic_shard_files(tmp_path):
    """Property check of the re-sharding reader: units with random padded sizes and random (equal
    or unequal) shard boundaries, files filled so that element i of tensor `which` of unit u holds
    u * 1e6 + which * 1e5 + i; any range read back must reproduce exactly those values."""
    import random

    import numpy as np

    from zorse_b200.ckpt.reader import _file_offsets, read_range

    rng = random.Random(0)
    for trial in range(20):
        d = tmp_path / f"t{trial}"
        d.mkdir()
        R = rng.randint(1, 4)
        ranks = rng.sample(range(16), R)
        units = []
        for gid in range(rng.randint(1, 5)):
            n = rng.randint(R, 40) * 8
            if rng.random() < 0.5:
                cuts = sorted(rng.sample(range(8, n, 8), R - 1)) if R > 1 and n // 8 > R else [n * (i + 1) // R // 8 * 8 for i in range(R - 1)]
                offs = [0] + cuts + [n]
                unit = {"stage": 0, "gid": gid, "numel": n - rng.randint(0, 7), "padded": n, "shard_ranks": ranks,
                        "shard_numel": max(b - a for a, b in zip(offs, offs[1:])), "shard_offsets": offs}
            else:
                n = (n // (8 * R)) * 8 * R or 8 * R
                unit = {"stage": 0, "gid": gid, "numel": n, "padded": n, "shard_ranks": ranks, "shard_numel": n // R}
            units.append(unit)
        meta = {"format_version": 1, "units": units}
        for idx, r in enumerate(ranks):
            blob = []
            for u in units:
                bd = u.get("shard_offsets") or [i * u["shard_numel"] for i in range(R + 1)]
                lo, hi = bd[idx], bd[idx + 1]
                for which in range(3):
                    blob.append((u["gid"] * 1e6 + which * 1e5 + np.arange(lo, hi)).astype("<f4").tobytes())
            (d / f"stage0_rank{r}.bin").write_bytes(b"".join(blob))
        offsets = _file_offsets(meta)
        for u in units:
            for _ in range(6):
                a = rng.randint(0, u["padded"] - 1)
                b = rng.randint(a + 1, u["padded"])
                which = rng.randint(0, 2)
                got = read_range(str(d), meta, offsets, u, which, a, b)
                want = torch.from_numpy((u["gid"] * 1e6 + which * 1e5 + np.arange(a, b)).astype("float32"))
                assert torch.equal(got, want), (trial, u, which, a, b)


def _resume_cli_like(rank, world, cfg_dict, ck):
    from zorse_b200.ckpt.reader import load_checkpoint
    from zorse_b200.trainer import Trainer, TrainerOptions

    tr = Trainer(parse_pipeline_dict(cfg_dict), TrainerOptions(backend="gloo", schedule="layer_major", seed=0))
    load_checkpoint(tr, ck)
    return tr.global_loss(tr.train_step_from_host(tr.synthetic_batch()))


def test_recover_replans_for_the_gpus_that_are_left(tmp_path):
    """A two-rank job saves, one GPU is lost: the recovery tool picks the newest complete checkpoint,
    drops the GPU from the cluster description, plans for the remaining one, and the job resumes
    there with the loss the old job would have had."""
    import json

    from zorse_b200.cli import recover

    ck = str(tmp_path / "ck")
    a = run_workers(2, _train_and_save, tiny_cfg(PIPE_1x2), ck, 2)
    os.makedirs(os.path.join(ck, "step_9"))                      # newer but incomplete: no meta.json
    assert recover.latest_checkpoint(ck) == os.path.join(ck, "step_2")
    assert recover.latest_checkpoint(str(tmp_path / "nothing")) is None
    assert recover.latest_checkpoint(ck, verify=True) == os.path.join(ck, "step_2")
    # a newer checkpoint with a cut-off shard file: named by the plain search, passed over by the verifying one
    import shutil
    shutil.copytree(os.path.join(ck, "step_2"), os.path.join(ck, "step_4"))
    with open(os.path.join(ck, "step_4", "stage0_rank1.bin"), "r+b") as fh:
        fh.truncate(100)
    assert recover.latest_checkpoint(ck) == os.path.join(ck, "step_4")
    assert recover.latest_checkpoint(ck, verify=True) == os.path.join(ck, "step_2")
    shutil.rmtree(os.path.join(ck, "step_4"))
    gl = [{"index": i, "name": "NVIDIA B200", "memory_total_mib": 183359, "id": f"gpu_{i}", "machine": "m0",
           "global_rank": i} for i in range(2)]
    cluster = {"machines": [{"machine": "m0", "num_gpus": 2, "machine_index": 0, "gpus": gl}], "gpu_list": gl,
               "total_gpus": 2, "bandwidth": {"internode_bandwidth": {}, "intranode_bandwidth": {"0": 770.0},
                                              "internode_latency": {}, "intranode_latency": {"0": 2e-5}}}
    small = recover.shrink_cluster(cluster, [0])
    assert small["total_gpus"] == 1 and small["gpu_list"][0]["global_rank"] == 0 and small["gpu_list"][0]["index"] == 1
    assert small["machines"][0]["num_gpus"] == 1 and cluster["total_gpus"] == 2       # the input is not modified
    with pytest.raises(ValueError):
        recover.shrink_cluster(cluster, [0, 1])
    with pytest.raises(ValueError):
        recover.shrink_cluster(cluster, [7])
    cfile, out = tmp_path / "cluster.json", tmp_path / "new.json"
    cfile.write_text(json.dumps(cluster))
    assert recover.main(["--checkpoint_dir", ck, "--cluster_info_file", str(cfile), "--exclude_ranks", "1",
                         "--output", str(out)]) == 0
    new = json.loads(out.read_text())
    cfg = parse_pipeline_dict(new)
    assert cfg.world_size == 1 and cfg.model_name == "tiny_llama" and cfg.global_batch_size == 8
    assert cfg.vocab_size == 512 and cfg.autocast_dtype == "float32"
    b = run_workers(1, _resume_cli_like, new, os.path.join(ck, "step_2"))
    assert abs(a[0] - b[0]) < 1e-4, (a, b)


def test_fault_injection_is_refused_where_a_leaving_rank_would_fault_its_peers():
    from zorse_b200.utils.health import injection_refusal

    assert injection_refusal(False, "fused", env={}) is None                       # CPU ranks: always allowed
    assert "NCCL_NVLS_ENABLE" in injection_refusal(True, "library", env={})
    assert "collectives" in injection_refusal(True, "fused", env={"NCCL_NVLS_ENABLE": "0"})
    assert "multimem" in injection_refusal(True, "library", env={"NCCL_NVLS_ENABLE": "0", "ZORSE_RS_ADAM_VARIANT": "3"})
    assert injection_refusal(True, "library", env={"NCCL_NVLS_ENABLE": "0"}) is None


def _masters_of(ck_dir):
    """gid -> whole fp32 master of every unit of a checkpoint, whatever plan wrote it."""
    from zorse_b200.ckpt.reader import _file_offsets, read_meta, read_range

    meta = read_meta(ck_dir)
    off = _file_offsets(meta)
    return meta["step"], {u["gid"]: read_range(ck_dir, meta, off, u, 0, 0, u["numel"]) for u in meta["units"]}


def test_supervised_job_survives_the_loss_of_a_rank(tmp_path):
    """End to end on CPU ranks: a 4-rank job (2 stages x 2) under the supervisor loses rank 1 before step 3 (the rank
    exits by itself, between steps); the supervisor blames that rank and not the peers that then fail on their
    connections, plans for the three GPUs that are left, resumes from the newest checkpoint and trains the remaining
    steps.  The final parameters equal those of the same job run without a failure."""
    import json

    from zorse_b200.cli import supervise

    gl = [{"index": i, "name": "NVIDIA B200", "memory_total_mib": 183359, "id": f"gpu_{i}", "machine": "m0",
           "global_rank": i} for i in range(4)]
    cluster = {"machines": [{"machine": "m0", "num_gpus": 4, "machine_index": 0, "gpus": gl}], "gpu_list": gl,
               "total_gpus": 4, "bandwidth": {"internode_bandwidth": {}, "intranode_bandwidth": {"0": 770.0},
                                              "internode_latency": {}, "intranode_latency": {"0": 2e-5}}}
    pipe = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [2, 2], "layer_partition": [0, 2], "zero_config": [[0, 1]]},
            {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [2, 2], "layer_partition": [2, 4], "zero_config": [[2, 3]]}]
    (tmp_path / "cluster.json").write_text(json.dumps(cluster))
    (tmp_path / "tc.json").write_text(json.dumps(tiny_cfg(pipe)))
    common = ["--config_file", str(tmp_path / "tc.json"), "--cluster_info_file", str(tmp_path / "cluster.json"),
              "--train_steps", "5", "--checkpoint_every", "1", "--max_restarts", "1", "--grace", "20"]
    trainer = ["--", "--backend", "gloo", "--skip_profile", "--lr", "1e-3"]
    assert supervise.main(common + ["--checkpoint_dir", str(tmp_path / "ck_a"), "--work_dir", str(tmp_path / "run_a")]
                          + trainer) == 0
    assert supervise.main(common + ["--checkpoint_dir", str(tmp_path / "ck_b"), "--work_dir", str(tmp_path / "run_b")]
                          + trainer + ["--inject_fault", "1:3:exit"]) == 0
    # the second job restarted once, on three ranks, from step 3
    new_cfg = parse_pipeline_dict(json.loads((tmp_path / "run_b" / "training_config_attempt1.json").read_text()))
    assert new_cfg.world_size == 3 and new_cfg.global_batch_size == 8
    assert (tmp_path / "run_b" / "attempt1_rank2.log").exists() and not (tmp_path / "run_b" / "attempt1_rank3.log").exists()
    assert "resumed from" in (tmp_path / "run_b" / "attempt1_rank0.log").read_text()
    sa, a = _masters_of(str(tmp_path / "ck_a" / "step_5"))
    sb, b = _masters_of(str(tmp_path / "ck_b" / "step_5"))
    assert sa == sb == 5 and set(a) == set(b)
    for gid in a:
        assert (a[gid] - b[gid]).abs().max().item() < 5e-5, gid
    # attribution rules on their own
    fr = supervise.failed_ranks
    assert fr({0: 1, 1: 17, 2: 1, 3: -15}, {0: "RuntimeError: Connection closed by peer", 1: "", 2: "recvBytes failed", 3: ""},
              [1, 0, 2, 3]) == [1]
    assert fr({0: 3, 1: -15, 2: 3}, {0: "[watchdog] rank 0: no progress for 9s; ranks behind or silent: [1]; dumping", 1: "",
                                     2: "[watchdog] rank 2: ...; ranks behind or silent: [1]"}, [0, 2, 1]) == [1]
    assert fr({0: 1, 1: 1}, {0: "Connection reset", 1: "Connection closed by peer"}, [1, 0]) == [1]
    # a stalled rank: everybody is "behind" (useless), but only rank 2 has not entered the step the others are in
    stuck = "[watchdog] rank {r}: no progress for 6.2s after step 2; ranks behind or silent: {b}; ranks that have not entered step 3: [2]"
    assert fr({0: 3, 1: -6, 2: -15, 3: 3}, {0: stuck.format(r=0, b=[1, 2, 3]), 1: "Connection closed by peer", 2: "",
                                            3: stuck.format(r=3, b=[0, 1, 2])}, [1, 0, 3, 2]) == [2]
    assert fr({0: 0, 1: 0}, {}, [0, 1]) == []


def _worker_message_fault(rank, world, cfg_dict, fault):
    """Step 0 runs clean; before step 1 rank 0 arms a message fault.  Returns (losses, error text or None, seconds)."""
    import time

    from zorse_b200.parallel.p2p import P2PTimeout
    from zorse_b200.trainer import Trainer, TrainerOptions
    from zorse_b200.utils.health import maybe_inject, parse_fault

    tr = Trainer(parse_pipeline_dict(cfg_dict), TrainerOptions(backend="gloo", schedule="1f1b", p2p_timeout_s=15.0,
                                                               p2p_fault_hooks=True))
    batch = tr.synthetic_batch()
    losses, err, t0 = [], None, time.time()
    for step in range(2):
        maybe_inject(parse_fault(fault), tr.rank, step, transport=tr.fault_transport)
        try:
            losses.append(tr.global_loss(tr.train_step_from_host(batch)))
        except (P2PTimeout, RuntimeError) as e:
            err = f"{type(e).__name__}: {e}"
            break
    return losses, err, time.time() - t0, list(tr.fault_transport.dropped)


def test_dropped_and_delayed_pipeline_messages():
    """Host-side message faults on Gloo ranks: a delayed activation only costs time; a dropped one ends the step on
    the receiving rank with an error that names the missing message (sender, tag, kind), within the receive limit,
    and the sender fails in bounded time too instead of waiting for ever."""
    from zorse_b200.utils.health import parse_fault

    cfg = tiny_cfg(PIPE_2x1)
    clean = run_workers(2, _worker_message_fault, cfg, None)
    late = run_workers(2, _worker_message_fault, cfg, "0:1:delay=1.5")
    assert [r[1] for r in late] == [None, None] and late[0][0] == pytest.approx(clean[0][0], abs=1e-6)
    assert late[0][2] > clean[0][2] + 1.0
    lost = run_workers(2, _worker_message_fault, cfg, "0:1:drop", timeout=180)
    (l0, e0, t0, d0), (l1, e1, t1, d1) = lost
    assert len(d0) == 1 and d0[0][0] == 1 and d0[0][2].startswith("act") and not d1
    assert e1 is not None and "P2PTimeout" in e1 and f"tag {d0[0][1]} from rank 0" in e1 and "act" in e1, e1
    assert e0 is not None and t0 < 120 and t1 < 120, (e0, t0, t1)
    assert len(l0) == 1 and len(l1) == 1 and l0[0] == pytest.approx(clean[0][0][0], abs=1e-6)     # step 0 was clean
    assert parse_fault("3:7:delay=0.5") == (3, 7, "delay=0.5")
    with pytest.raises(ValueError):
        parse_fault("0:1:lose")


def test_supervised_job_survives_a_rank_that_stalls(tmp_path):
    """A rank that stops between steps without exiting (it never joins step 3): the peers' watchdogs end them and
    report who never entered the step they are stuck in; the supervisor ends the silent rank, restarts on the other
    three from the newest checkpoint and the job reaches its last step."""
    import json

    from zorse_b200.cli import supervise

    gl = [{"index": i, "name": "NVIDIA B200", "memory_total_mib": 183359, "id": f"gpu_{i}", "machine": "m0",
           "global_rank": i} for i in range(4)]
    cluster = {"machines": [{"machine": "m0", "num_gpus": 4, "machine_index": 0, "gpus": gl}], "gpu_list": gl,
               "total_gpus": 4, "bandwidth": {"internode_bandwidth": {}, "intranode_bandwidth": {"0": 770.0},
                                              "internode_latency": {}, "intranode_latency": {"0": 2e-5}}}
    pipe = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [2, 2], "layer_partition": [0, 2], "zero_config": [[0, 1]]},
            {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [2, 2], "layer_partition": [2, 4], "zero_config": [[2, 3]]}]
    (tmp_path / "cluster.json").write_text(json.dumps(cluster))
    (tmp_path / "tc.json").write_text(json.dumps(tiny_cfg(pipe)))
    rc = supervise.main(["--config_file", str(tmp_path / "tc.json"), "--cluster_info_file", str(tmp_path / "cluster.json"),
                         "--train_steps", "5", "--checkpoint_every", "1", "--max_restarts", "1", "--grace", "12",
                         "--checkpoint_dir", str(tmp_path / "ck"), "--work_dir", str(tmp_path / "run"),
                         "--", "--backend", "gloo", "--skip_profile", "--heartbeat_timeout", "6", "--heartbeat_startup", "90",
                         "--inject_fault", "2:3:stall"])
    assert rc == 0
    logs = "".join((tmp_path / "run" / f"attempt0_rank{r}.log").read_text() for r in (0, 1, 3))
    assert "ranks that have not entered step 3: [2]" in logs
    new_cfg = parse_pipeline_dict(json.loads((tmp_path / "run" / "training_config_attempt1.json").read_text()))
    assert new_cfg.world_size == 3
    step, _ = _masters_of(str(tmp_path / "ck" / "step_5"))
    assert step == 5
