"""Distributed plumbing on CPU ranks (gloo): every stage split / DP width / schedule must
reproduce the single-process oracle trainer (same loss, same parameters after two steps)."""
import pytest
import torch

from dist_utils import run_workers
from zorse_b200.config.training_config import parse_pipeline_dict


def tiny_cfg(pipeline, gbs=8, mbs=2, seq=32, vocab=512, **kw):
    d = {"model_name": "tiny_llama", "global_batch_size": gbs, "microbatch_size": mbs, "sequence_length": seq,
         "vocab_size": vocab, "autocast_dtype": "float32", "reduce_dtype": "float32", "pipeline_config": pipeline}
    d.update(kw)
    return d


def _worker(rank, world, cfg_dict, opts, steps):
    from zorse_b200.trainer import Trainer, TrainerOptions

    cfg = parse_pipeline_dict(cfg_dict)
    tr = Trainer(cfg, TrainerOptions(backend="gloo", **opts))
    batch = tr.synthetic_batch()
    losses = []
    for _ in range(steps):
        loss = tr.train_step_from_host(batch)
        losses.append(tr.global_loss(loss))
    params = {}
    for st in tr.stages:
        for u in st.engine.units:
            params[u.gid] = u.full_master()[: u.layer.layout()[1]].clone()
    cnt = [(c.all_gathers, c.reduce_scatters, c.all_reduces, c.adam_steps) for c in tr.counters()]
    return {"losses": losses, "params": params, "counters": cnt}


def _oracle(cfg_dict, steps):
    from zorse_b200.utils.oracle import OracleTrainer

    cfg = parse_pipeline_dict(cfg_dict)
    orc = OracleTrainer(cfg)
    g = torch.Generator().manual_seed(7919)
    M, B, S = cfg.num_microbatches, cfg.microbatch_size, cfg.sequence_length
    batch = {"inputs": torch.randint(0, cfg.vocab_size, (M, B, S), generator=g),
             "targets": torch.randint(0, cfg.vocab_size, (M, B, S), generator=g)}
    losses = [orc.step(batch) for _ in range(steps)]
    return losses, [f.detach() for f in orc.flats]


def _check(results, cfg_dict, steps=2, ptol=5e-4):
    want_losses, want_params = _oracle(cfg_dict, steps)
    for res in results:
        for a, b in zip(res["losses"], want_losses):
            assert abs(a - b) < 2e-4, (res["losses"], want_losses)
        for gid, p in res["params"].items():
            err = (p - want_params[gid]).abs().max().item()
            assert err < ptol, f"unit {gid}: max param error {err}"


PIPE_2x1 = [{"gpu_ranks": [0], "num_microbatches_per_rank": [4], "layer_partition": [0, 2], "zero_config": [[0]]},
            {"gpu_ranks": [1], "num_microbatches_per_rank": [4], "layer_partition": [2, 4], "zero_config": [[1]]}]
PIPE_1x2 = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [2, 2], "layer_partition": [0, 4],
             "zero_config": [[0, 1]]}]
PIPE_1x2_UNEVEN = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [3, 1], "layer_partition": [0, 4],
                    "zero_config": [[0, 1]]}]


@pytest.mark.parametrize("schedule", ["layer_major", "zero2", "1f1b", "no_overlap", "two_stage_sync", "flashflex"])
def test_two_stages_one_dp(schedule):
    """Benchmark configuration 1: tiny Llama, 2 stages x 1 DP over gloo."""
    cfg = tiny_cfg(PIPE_2x1)
    res = run_workers(2, _worker, cfg, {"schedule": schedule}, 2)
    _check(res, cfg)


@pytest.mark.parametrize("schedule,oib", [("layer_major", False), ("layer_major", True), ("zero2", True), ("1f1b", False)])
def test_one_stage_two_dp(schedule, oib):
    cfg = tiny_cfg(PIPE_1x2)
    res = run_workers(2, _worker, cfg, {"schedule": schedule, "optimizer_in_backward": oib}, 2)
    _check(res, cfg)
    # layer-major ZeRO-3: each unit gathered twice per step (forward, backward) and reduced once
    ag, rs, ar, adam = res[0]["counters"][0]
    n_units = 6
    assert rs == 2 * n_units and adam == 2 * n_units
    if schedule == "layer_major":
        assert ag == 2 * (2 * n_units - 1)


def test_uneven_microbatches_per_rank():
    cfg = tiny_cfg(PIPE_1x2_UNEVEN)
    res = run_workers(2, _worker, cfg, {"schedule": "layer_major"}, 2)
    _check(res, cfg)


@pytest.mark.parametrize("schedule,oib", [("layer_major", False), ("zero2", True)])
def test_uneven_parameter_shards(schedule, oib):
    """Rank 0 owns about 70 % of every unit: broadcast-per-owner gather and reduce-per-owner
    reduction must give the same training as equal shards."""
    pipe = [dict(PIPE_1x2[0], shard_ratio=[0.7, 0.3])]
    cfg = tiny_cfg(pipe)
    res = run_workers(2, _worker, cfg, {"schedule": schedule, "optimizer_in_backward": oib}, 2)
    _check(res, cfg)


def test_shard_bounds():
    from zorse_b200.engine.zero import shard_bounds
    from zorse_b200.models.layers import ALIGN

    n = 64 * ALIGN
    assert shard_bounds(n, 4) == [0, n // 4, n // 2, 3 * n // 4, n]
    b = shard_bounds(n, 3, [2, 1, 1])
    assert b[0] == 0 and b[-1] == n and all(x % ALIGN == 0 for x in b)
    assert b[1] == n // 2 and b[2] == 3 * n // 4
    tiny = shard_bounds(4 * ALIGN, 4, [1000, 1, 1, 1])      # every rank keeps at least one block
    assert all(tiny[i + 1] - tiny[i] >= ALIGN for i in range(4))
    with pytest.raises(ValueError):
        shard_bounds(n, 2, [1.0])


def test_offload_params():
    cfg = tiny_cfg(PIPE_1x2)
    res = run_workers(2, _worker, cfg, {"schedule": "zero2", "optimizer_in_backward": True,
                                        "offload_model_params": True}, 2)
    _check(res, cfg)


@pytest.mark.parametrize("schedule", ["layer_major", "zero2", "1f1b"])
def test_mixed_widths_and_hybrid(schedule):
    """4 ranks: stage 0 on one... two ranks (2-way shard), stage 1 on two ranks as two
    replicate groups of one (hybrid: all-reduce only), uneven microbatch counts."""
    pipe = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [3, 1], "layer_partition": [0, 1], "zero_config": [[0, 1]]},
            {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [1, 3], "layer_partition": [1, 4], "zero_config": [[2], [3]]}]
    cfg = tiny_cfg(pipe)
    res = run_workers(4, _worker, cfg, {"schedule": schedule}, 2)
    _check(res, cfg)


@pytest.mark.parametrize("schedule", ["zero2", "1f1b"])
def test_latency_driven_routing_trains_like_the_oracle(schedule):
    """The same 4-rank plan with the microbatches routed by per-rank latencies (a slow rank on each stage): the
    routing changes who carries which microbatch, not the result."""
    pipe = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [3, 1], "layer_partition": [0, 1], "zero_config": [[0, 1]]},
            {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [1, 3], "layer_partition": [1, 4], "zero_config": [[2], [3]]}]
    cfg = tiny_cfg(pipe)
    cfg["comm_plan"] = "latency"
    cfg["rank_latency_ms"] = {"0": 1.0, "1": 2.5, "2": 3.0, "3": 1.0}
    res = run_workers(4, _worker, cfg, {"schedule": schedule}, 2)
    _check(res, cfg)


def test_interleaved_stages_three_ranks():
    """1 -> 2 -> 1 widths with rank 0 hosting the first and the last stage."""
    pipe = [{"gpu_ranks": [0], "num_microbatches_per_rank": [4], "layer_partition": [0, 1], "zero_config": [[0]]},
            {"gpu_ranks": [1, 2], "num_microbatches_per_rank": [2, 2], "layer_partition": [1, 3], "zero_config": [[1, 2]]},
            {"gpu_ranks": [0], "num_microbatches_per_rank": [4], "layer_partition": [3, 4], "zero_config": [[0]]}]
    cfg = tiny_cfg(pipe)
    res = run_workers(3, _worker, cfg, {"schedule": "layer_major"}, 2)
    _check(res, cfg)


def test_trainer_cli_end_to_end(tmp_path):
    """`zorse.py` under torchrun on two gloo ranks: flags of the reference plus the debug aids,
    summary block with the CSV header scripts parse, checkpoint written and resumable."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = tiny_cfg(PIPE_2x1, fused_optimizer=True)
    cfg_file = tmp_path / "training_config.json"
    cfg_file.write_text(json.dumps(cfg))
    ck = tmp_path / "ck"
    base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
            "127.0.0.1", "--master-port", "29877", os.path.join(root, "zorse.py"), "--config_file", str(cfg_file),
            "--backend", "gloo", "--ops", "ref", "--iterations", "2", "--warmup_iterations", "3", "--skip_profile"]
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run(base + ["--zero2_pipeline", "--optimizer_in_backwards", "--replay_check", "--nvtx",
                               "--checkpoint_dir", str(ck), "--checkpoint_every", "5"],
                       capture_output=True, text=True, timeout=300, env=env, cwd=root)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "replay check: identical=True" in out
    assert "Throughput:" in out and "Batch Size,Seq_Len,Min_Allocated,Max_Allocated,Latency,Throughput" in out
    assert (ck / "step_5" / "meta.json").exists()
    assert out.count("===== zorse-b200 run summary =====") == 1
    # resumed, with the summary after every timed iteration (two of them: one running block + the final one)
    r2 = subprocess.run(base + ["--resume", str(ck / "step_5"), "--print_metrics_every_iteration"], capture_output=True,
                        text=True, timeout=300, env=env, cwd=root)
    out2 = r2.stdout + r2.stderr
    assert r2.returncode == 0, out2[-3000:]
    assert out2.count("===== zorse-b200 run summary =====") == 2 and "resumed from" in out2


def _interleaved_pipe(P, v, width, M):
    pipe = []
    for k in range(P * v):
        ranks = list(range((k % P) * width, (k % P + 1) * width))
        pipe.append({"gpu_ranks": ranks, "num_microbatches_per_rank": [M // width] * width,
                     "layer_partition": [k, k + 1], "zero_config": [ranks]})
    return pipe


@pytest.mark.parametrize("P,v,width,M", [(2, 2, 1, 4), (2, 2, 2, 8)])
def test_interleaved_1f1b(P, v, width, M):
    """Two model chunks per rank (stages g and g + P): same training as the oracle."""
    cfg = tiny_cfg(_interleaved_pipe(P, v, width, M), gbs=M, mbs=1)
    res = run_workers(P * width, _worker, cfg, {"schedule": "1f1b_interleaved"}, 2)
    _check(res, cfg)


def test_interleaved_1f1b_rejects_bad_plans():
    from zorse_b200.parallel.p2p_sim import record_programs

    cfg = parse_pipeline_dict(tiny_cfg(_interleaved_pipe(2, 2, 1, 3), gbs=3, mbs=1))   # 3 microbatches, 2 groups
    with pytest.raises(ValueError, match="multiple of 2 rank groups"):
        record_programs(cfg, "1f1b_interleaved")


def test_idle_rank_left_out_by_the_planner():
    """A plan that gives a slow GPU no stage: that rank still joins the job (groups, barriers, loss
    reduction) and idles; the other ranks train as the oracle does."""
    pipe = [{"gpu_ranks": [0], "num_microbatches_per_rank": [4], "layer_partition": [0, 2], "zero_config": [[0]]},
            {"gpu_ranks": [2], "num_microbatches_per_rank": [4], "layer_partition": [2, 4], "zero_config": [[2]]}]
    cfg = tiny_cfg(pipe, unused_ranks=[1])
    assert parse_pipeline_dict(cfg).world_size == 3
    res = run_workers(3, _worker, cfg, {"schedule": "zero2"}, 2)
    assert res[1]["params"] == {} and res[1]["counters"] == []
    _check(res, cfg)
    with pytest.raises(ValueError, match="0 .. world_size - 1"):
        parse_pipeline_dict(tiny_cfg(pipe))            # rank 1 missing and not declared idle


@pytest.mark.parametrize("schedule", ["zero2", "1f1b"])
def test_rank_without_microbatches_joins_reductions_in_peer_order(schedule):
    """Stage 0 has two replicas of which one runs no microbatch at all (a very slow GPU): it must
    still take part in every gradient all-reduce, in the same layer order as its peer."""
    pipe = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [0, 4], "layer_partition": [0, 1], "zero_config": [[0], [1]]},
            {"gpu_ranks": [2], "num_microbatches_per_rank": [4], "layer_partition": [1, 2], "zero_config": [[2]]},
            {"gpu_ranks": [3, 4], "num_microbatches_per_rank": [3, 1], "layer_partition": [2, 4], "zero_config": [[3], [4]]}]
    cfg = tiny_cfg(pipe, gbs=8, mbs=2)
    res = run_workers(5, _worker, cfg, {"schedule": schedule}, 2)
    _check(res, cfg)


@pytest.mark.parametrize("schedule", ["layer_major", "zero2"])
def test_consecutive_stages_on_the_same_ranks(schedule):
    """Two stages on one rank group (an interleaved plan with a single group): a microbatch's next
    owner can be the sending rank itself; such hand-offs stay local instead of going through a
    transport that cannot send to itself."""
    pipe = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [1, 3], "layer_partition": [0, 2], "zero_config": [[0, 1]]},
            {"gpu_ranks": [0, 1], "num_microbatches_per_rank": [1, 3], "layer_partition": [2, 4], "zero_config": [[0, 1]]}]
    cfg = tiny_cfg(pipe, gbs=8, mbs=2)
    res = run_workers(2, _worker, cfg, {"schedule": schedule, "optimizer_in_backward": True}, 2)
    _check(res, cfg)


@pytest.mark.parametrize("schedule,pipe_name", [("1f1b", "PIPE_2x1"), ("1f1b_interleaved", "INTERLEAVED")])
def test_deferred_weight_gradients_give_the_same_training(schedule, pipe_name):
    """Sending a microbatch's input gradient upstream before its weight-gradient GEMMs run reorders work
    only: losses and parameters still match the oracle, and the hold-back really happened."""
    if pipe_name == "PIPE_2x1":
        pipe = PIPE_2x1
    else:
        pipe = [{"gpu_ranks": [k % 2], "num_microbatches_per_rank": [4], "layer_partition": [k, k + 1],
                 "zero_config": [[k % 2]]} for k in range(4)]
    cfg = tiny_cfg(pipe)
    res = run_workers(2, _worker_defer, cfg, {"schedule": schedule, "defer_wgrad": True}, 2)
    _check([r["result"] for r in res], cfg)
    assert any(r["deferred"] > 0 for r in res), [r["deferred"] for r in res]
    if pipe_name == "PIPE_2x1":
        assert res[0]["deferred"] == 0        # the first stage sends nothing upstream: nothing to gain there


def _worker_defer(rank, world, cfg_dict, opts, steps):
    from zorse_b200.parallel.stage import DeferredWgrad

    count = {"n": 0}
    orig = DeferredWgrad.flush

    def counting_flush(self):
        count["n"] += len(self._queue)
        return orig(self)

    DeferredWgrad.flush = counting_flush
    try:
        return {"result": _worker(rank, world, cfg_dict, opts, steps), "deferred": count["n"]}
    finally:
        DeferredWgrad.flush = orig


@pytest.mark.parametrize("pipe_name,k", [("PIPE_2x1", 1), ("PIPE_2x1", 2), ("MIXED", 2), ("PIPE_1x2_UNEVEN", 2)])
def test_tail_deferred_weight_gradients_give_the_same_training(pipe_name, k):
    """1F1B with the last stage's head (k = 1) or head + last block (k = 2) weight gradients held back until the
    stage's last backward: same losses and parameters as the oracle (two stages x 1, and two stages x 2-way shard with
    uneven microbatch counts, where a reduction order shared by the stage's ranks matters; one stage x 2: allowed,
    pointless)."""
    mixed = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [3, 1], "layer_partition": [0, 2], "zero_config": [[0, 1]]},
             {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [1, 3], "layer_partition": [2, 4], "zero_config": [[2, 3]]}]
    pipe = {"PIPE_2x1": PIPE_2x1, "PIPE_1x2_UNEVEN": PIPE_1x2_UNEVEN}.get(pipe_name, mixed)
    # k = 1 on the two-stage plan comes from the config file's key, the others from the trainer option
    by_key = pipe_name == "PIPE_2x1" and k == 1
    cfg = tiny_cfg(pipe, **({"defer_tail_wgrad": k} if by_key else {}))
    opts = {"schedule": "1f1b"} if by_key else {"schedule": "1f1b", "defer_tail_wgrad": k}
    res = run_workers(4 if pipe_name == "MIXED" else 2, _worker_defer, cfg, opts, 2)
    _check([r["result"] for r in res], cfg)
    if pipe_name == "PIPE_2x1":
        # the last stage's rank held back one GEMM (head) or five (head + the block's four) per microbatch and step
        assert [r["deferred"] for r in res] == [0, 2 * 4 * (1 if k == 1 else 5)]


@pytest.mark.parametrize("pipe_name", ["PIPE_2x1", "CHAIN4", "MIXED"])
def test_1f1b_with_preposted_receives_gives_the_same_training(pipe_name):
    """Receives posted one operation ahead (`prepost_recv`, per-boundary groups): two stages, a chain of four stages
    (middle ranks hold two receives in flight) and two stages x 2 with uneven counts all match the oracle."""
    chain4 = [{"gpu_ranks": [k], "num_microbatches_per_rank": [4], "layer_partition": [k, k + 1], "zero_config": [[k]]}
              for k in range(4)]
    mixed = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [3, 1], "layer_partition": [0, 2], "zero_config": [[0, 1]]},
             {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [1, 3], "layer_partition": [2, 4], "zero_config": [[2, 3]]}]
    pipe = {"PIPE_2x1": PIPE_2x1, "CHAIN4": chain4, "MIXED": mixed}[pipe_name]
    cfg = tiny_cfg(pipe)
    res = run_workers(2 if pipe_name == "PIPE_2x1" else 4, _worker, cfg, {"schedule": "1f1b", "prepost_recv": True}, 2)
    _check(res, cfg)


def _worker_patterns(rank, world):
    """Every collective pattern once on 4 gloo ranks arranged as 2 nodes x 2: results on all-ones inputs."""
    import torch.distributed as dist

    from zorse_b200.parallel.groups import dist_init
    from zorse_b200.profiler import collectives as C

    dist_init("gloo")
    dev, f32 = torch.device("cpu"), torch.float32
    groups = C.node_groups(local_size=2)
    intra, inter = groups
    assert dist.get_process_group_ranks(intra) == [rank // 2 * 2, rank // 2 * 2 + 1]
    assert dist.get_process_group_ranks(inter) == [rank % 2, rank % 2 + 2]
    out = {}
    n = 64
    p = C.AllReduce(n, f32, device=dev); p.execute(); out["all_reduce"] = float(p.full[0])
    p = C.AllGather(n, f32, device=dev); p.execute(); out["all_gather"] = (p.full.numel(), float(p.full.sum()))
    p = C.ReduceScatter(n, f32, device=dev); p.execute(); out["reduce_scatter"] = (p.shard.numel(), float(p.shard[0]))
    p = C.Broadcast(n, f32, device=dev); p.execute(); out["broadcast"] = float(p.full[0])
    p = C.IntraNodeAllGather(n, f32, dev, groups); p.execute(); out["intra_ag"] = (p.name, p.shard.numel(), p.full.numel())
    p = C.InterNodeAllGather(n, f32, dev, groups); p.execute(); out["inter_ag"] = (p.name, p.shard.numel(), p.full.numel())
    p = C.IntraNodeReduceScatter(n, f32, dev, groups); p.execute(); out["intra_rs"] = (p.name, float(p.shard[0]))
    p = C.InterNodeReduceScatter(n, f32, dev, groups); p.execute(); out["inter_rs"] = (p.name, float(p.shard[0]))
    p = C.HybridReduceScatter(n, f32, intra, inter, dev); p.execute(); out["hybrid"] = (p.shard.numel(), float(p.shard[0]))
    p = C.ReduceScatter2Hop(n, f32, intra, inter, dev); p.execute()
    out["two_hop"] = (p.name, p.shard2.numel(), float(p.shard2[0]), float(p.shard[0]))
    p = C.Zero25(n, f32, intra, inter, dev); p.execute(); out["zero25"] = (p.name, float(p.shard[0]), float(p.shard[-1]))
    p = C.Zero25Global(n, f32, device=dev); p.execute(); out["zero25g"] = (p.name, float(p.full[0]), float(p.full[-1]))
    p = C.UnevenAllGather(n, [4, 2, 1, 1], f32, device=dev); p.execute(); out["uneven_ag"] = [t.numel() for t in p.parts]
    p = C.UnevenReduceScatter(n, None, f32, device=dev, sizes=[10, 20, 30, 4]); p.execute()
    out["uneven_rs"] = (p.mine.numel(), float(p.mine[0]))
    t = C.time_pattern(C.Zero25(n, f32, intra, inter, dev), warmup=1, trials=2)
    out["timed"] = sorted(t)
    return out


def test_collective_patterns_on_two_by_two_gloo_ranks():
    """The benchmark patterns (world-wide, per node, across nodes, hybrid, 2-hop with and without the gather back,
    list-based) compute what their names say (reference utils/comm_patterns.py)."""
    res = run_workers(4, _worker_patterns)
    for r, o in enumerate(res):
        assert o["all_reduce"] == 4.0 and o["all_gather"] == (64, 64.0) and o["reduce_scatter"] == (16, 4.0)
        assert o["broadcast"] == 1.0
        assert o["intra_ag"] == ("intra_node_all_gather", 16, 32) and o["inter_ag"] == ("inter_node_all_gather", 16, 32)
        assert o["intra_rs"] == ("intra_node_reduce_scatter", 2.0) and o["inter_rs"] == ("inter_node_reduce_scatter", 2.0)
        assert o["hybrid"] == (32, 4.0)                     # summed over the node, then over the nodes
        assert o["two_hop"] == ("reduce_scatter_2hop", 16, 4.0, 2.0)       # outer shard fully reduced, inner shard not
        assert o["zero25"] == ("zero_2_5", 4.0, 4.0)                         # gathered back: whole inner shard reduced
        assert o["zero25g"] == ("zero_2_5_global", 4.0, 4.0)
        assert o["uneven_ag"] == [32, 16, 8, 8]
        assert o["uneven_rs"] == ([10, 20, 30, 4][r], 4.0)
        assert {"avg_time_ms", "bandwidth_mbps", "world_size"} <= set(o["timed"])
