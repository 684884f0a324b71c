"""Config parsing/validation, static p2p plans, planner arithmetic, comm model, file formats."""
import json
import math
import os

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from zorse_b200.config import training_config as tc
from zorse_b200.models import registry
from zorse_b200.parallel.p2p_plan import create_static_comm_plans, interleave_owners
from zorse_b200.planner import comm_model as cm
from zorse_b200.planner.cluster import GPU, GPUGroup, ModelConfig, ModelLatencies
from zorse_b200.planner.memory import group_memory_bytes
from zorse_b200.planner.stage2 import PipelineOptimizer, distribute_layers, distribute_microbatches

REF_EXAMPLE = {
    "model_name": "deepspeedllama_tiny", "global_batch_size": 128, "microbatch_size": 2, "sequence_length": 512,
    "vocab_size": 49152, "fused_optimizer": True, "interleave_degree": 1, "latency": 7721.375000533334,
    "autocast_dtype": "float16", "reduce_dtype": "float32",
    "pipeline_config": [{"gpu_ranks": [0, 3, 2, 1], "num_microbatches_per_rank": [18, 1, 28, 17],
                         "layer_partition": [0, 22], "zero_config": [[0, 3, 2, 1]]}]}


def test_reference_example_round_trip():
    cfg = tc.parse_pipeline_dict(REF_EXAMPLE)
    assert cfg.num_microbatches == 64 and cfg.stages[0].num_microbatches_per_rank == (18, 1, 28, 17)
    assert cfg.gloo_batch_recv and cfg.alternate_nccl_gloo and not cfg.sync_after_recompute
    again = tc.parse_pipeline_dict(json.loads(json.dumps(tc.to_dict(cfg))))
    assert tc.to_dict(again) == tc.to_dict(cfg)
    assert tc.to_dict(cfg)["latency"] == REF_EXAMPLE["latency"]


def test_shipped_example_configs_parse():
    """Every training config under example/ parses, and the CPU one is the two-stage plan of the first benchmark
    configuration (tiny decoder: 4 layers, hidden 512, 8 heads, FFN 1376, vocabulary 32000, fp32)."""
    import glob
    import os

    from zorse_b200.models import registry

    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "example")
    files = sorted(glob.glob(os.path.join(root, "training_config*.json")))
    assert len(files) >= 2
    for f in files:
        tc.parse_pipeline_config(f)
    cpu = tc.parse_pipeline_config(os.path.join(root, "training_config_cpu_2stage.json"))
    spec = registry.get_spec(cpu.model_name)
    assert (spec.layers, spec.hidden, spec.heads, spec.ffn) == (4, 512, 8, 1376)
    assert (cpu.global_batch_size, cpu.microbatch_size, cpu.sequence_length, cpu.vocab_size) == (8, 2, 128, 32000)
    assert [s.gpu_ranks for s in cpu.stages] == [(0,), (1,)] and cpu.autocast_dtype == "float32"


@pytest.mark.parametrize("mutate,msg", [
    (lambda d: d["pipeline_config"][0].update(layer_partition=[1, 22]), "starts at"),
    (lambda d: d["pipeline_config"][0].update(num_microbatches_per_rank=[1, 1, 1, 1]), "microbatches"),
    (lambda d: d["pipeline_config"][0].update(zero_config=[[0, 3], [2]]), "partition|sizes"),
    (lambda d: d.update(global_batch_size=127), "multiple"),
    (lambda d: d.update(autocast_dtype="int8"), "dtype"),
    (lambda d: d.pop("model_name"), "required"),
])
def test_config_validation_errors(mutate, msg):
    d = json.loads(json.dumps(REF_EXAMPLE))
    mutate(d)
    with pytest.raises(tc.ConfigError, match=msg):
        tc.parse_pipeline_dict(d)


def test_stage_sorting_gaps_and_even_split():
    d = json.loads(json.dumps(REF_EXAMPLE))
    d["split_microbatches_evenly"] = True
    d["pipeline_config"] = [
        {"gpu_ranks": [2, 3], "layer_partition": [10, 22], "zero_config": [[2], [3]]},
        {"gpu_ranks": [0, 1], "layer_partition": [0, 10], "zero_config": [[0, 1]]}]
    cfg = tc.parse_pipeline_dict(d)
    assert [s.layer_partition for s in cfg.stages] == [(0, 10), (10, 22)]
    assert cfg.stages[0].num_microbatches_per_rank == (32, 32)
    assert cfg.stages[1].replicate_group_of(3) == (2, 3) and cfg.stages[1].shard_group_of(3) == (3,)
    d["pipeline_config"][0]["layer_partition"] = [11, 22]
    with pytest.raises(tc.ConfigError, match="contiguous"):
        tc.parse_pipeline_dict(d)


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(0, 9), min_size=1, max_size=5).filter(lambda c: sum(c) > 0))
def test_interleave_owners_counts(counts):
    own = interleave_owners(counts)
    assert len(own) == sum(counts)
    assert [own.count(k) for k in range(len(counts))] == list(counts)


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 3), st.integers(1, 3), st.integers(1, 3), st.integers(2, 12), st.data())
def test_static_plan_invariants(w0, w1, w2, M, data):
    widths = [w0, w1, w2]
    pipe, rank, bounds = [], 0, [0, 2, 3, 4]
    for i, w in enumerate(widths):
        ranks = list(range(rank, rank + w))
        rank += w
        cuts = sorted(data.draw(st.lists(st.integers(0, M), min_size=w - 1, max_size=w - 1)))
        counts = [b - a for a, b in zip([0] + cuts, cuts + [M])]
        pipe.append({"gpu_ranks": ranks, "num_microbatches_per_rank": counts, "layer_partition": [bounds[i], bounds[i + 1]],
                     "zero_config": [ranks]})
    cfg = tc.parse_pipeline_dict({"model_name": "tiny_llama", "global_batch_size": M, "microbatch_size": 1,
                                  "sequence_length": 8, "pipeline_config": pipe})
    plans = create_static_comm_plans(cfg)  # validates: each transfer once, mirrored, unique tags
    assert sorted(plans) == list(range(rank))
    for st_cfg in cfg.stages:
        got = sorted(g for r in st_cfg.gpu_ranks for g in plans[r].stages[st_cfg.stage_id].microbatches)
        assert got == list(range(M))


@settings(max_examples=50, deadline=None)
@given(st.integers(1, 200), st.lists(st.floats(0.5, 50.0), min_size=1, max_size=8))
def test_distribution_sum_rules(total, lat):
    m = distribute_microbatches(total, lat)
    assert sum(m) == total and all(x >= 0 for x in m)
    fastest, slowest = lat.index(min(lat)), lat.index(max(lat))
    assert m[fastest] >= m[slowest]
    L = distribute_layers(total, lat)
    assert sum(L) == total and L[fastest] >= L[slowest]


def _groups(n_groups, per_group, ag=1.0):
    out, r = [], 0
    for g in range(n_groups):
        gp = [GPU("b200", r + i) for i in range(per_group)]
        r += per_group
        out.append(GPUGroup(g, gp, ag, ag, 0.05, 0.05))
    return out


def test_optimizer_latency_monotone_and_uneven_split():
    model = ModelConfig("llama2_7b", 32, 4096, 202383360, 6738415616, 4096, 64)
    lat = {"b200": ModelLatencies(2.0, 4.0)}
    opt = PipelineOptimizer(_groups(4, 2), model, lat, 1)
    res = opt.optimize()
    assert res is not None and sum(s.num_layers for s in res.stages) == 32
    slow = PipelineOptimizer(_groups(4, 2), model, {"b200": ModelLatencies(4.0, 8.0)}, 1).optimize()
    assert slow.latency_ms > res.latency_ms
    # a slower group gets fewer layers
    groups = _groups(2, 4)
    groups[1].gpus = [GPU("h100", 4 + i) for i in range(4)]
    res2 = PipelineOptimizer(groups, model, {"b200": ModelLatencies(2.0, 4.0), "h100": ModelLatencies(4.0, 9.0)}, 1,
                             max_interleave=1).optimize()
    n = {s.group_id: s.num_layers for s in res2.stages}
    assert n[0] > n[1] and n[0] + n[1] == 32
    # interleaving keeps every layer exactly once and each group's total
    st2 = opt.interleave(opt.generate_stage_configs()[0], 2)
    assert [s.layer_partition[0] for s in st2] == sorted(s.layer_partition[0] for s in st2)
    assert st2[-1].layer_partition[1] == 32 and len(st2) == 8


def test_memory_model_and_comm_model():
    one = group_memory_bytes([8], 2, 202383360, 1, 4096, 4096)
    two = group_memory_bytes([4, 4], 2, 202383360, 1, 4096, 4096)
    assert math.isclose(one, two)  # maxpair covers all 8 layers in both
    assert group_memory_bytes([8], 4, 202383360, 1, 4096, 4096) < one
    bw = [[0, 10.0], [10.0, 0]]
    size = 1e9
    assert math.isclose(cm.ring_collective_ms(size, bw), 0.5 * 1.0 / 10 * 1e3)
    assert math.isclose(cm.ring_collective_ms_v2(size, bw), 1.15 * 0.5 / 10 * 1e3)
    assert math.isclose(cm.switch_collective_ms(size, 2, 0.02, 700.0), 0.02 + 0.5 / 700 * 1e3)
    assert cm.p2p_ms(5e6, 10.0, 0.004) == pytest.approx(4.0 * 0.9)
    assert cm.p2p_ms(2e7, 10.0, 0.004) == pytest.approx(4.0 + 1.0)


def test_model_registry_parameter_counts():
    # per-layer counts published in the reference's data/model_stats.json
    for name, per_layer in [("deepspeedllama_7b", 202383360), ("deepspeedllama_tiny", 51384320),
                            ("deepspeedllama_3b", 123910400), ("deepspeedllama_13b", 317204480),
                            ("deepspeedllama_65b", 809517056)]:
        assert registry.get_model_stats(name)["parameters_per_layer"] == per_layer
    assert registry.get_model_stats("deepspeedllama_7b", vocab=49152)["total_parameters"] == 6878924800
    assert registry.get_config_for_model("deepspeedllama_13b") == (40, 5120, 40, 13824)
    s = registry.get_spec("llama3.2_1b")
    assert (s.n_kv, s.head_dim, s.vocab) == (8, 64, 128256)
    with pytest.raises(ValueError, match="Unsupported model"):
        registry.get_spec("nope")
    layers = registry.build_stage_layers(registry.get_spec("tiny_llama"), 2, 4, 128)
    assert [l.kind for l in layers] == ["block", "block", "head"]


def test_planner_end_to_end(tmp_path):
    from zorse_b200.planner.plan import export_config, plan

    gl = [{"index": i, "name": "NVIDIA B200", "memory_total_mib": 183359, "id": f"gpu_{i}", "machine": "m0",
           "global_rank": i} for i in range(8)]
    data = {"machines": [{"machine": "m0", "num_gpus": 8, "machine_index": 0, "gpus": gl}], "gpu_list": gl,
            "total_gpus": 8, "bandwidth": {"internode_bandwidth": {}, "intranode_bandwidth": {"0": 770.0},
                                           "internode_latency": {}, "intranode_latency": {"0": 2e-5}},
            "collective_fit": {"all_gather": {"2": {"alpha_ms": 0.03, "bandwidth_gbs": 650.0}},
                               "reduce_scatter": {"2": {"alpha_ms": 0.03, "bandwidth_gbs": 650.0}}}}
    res, tried = plan(data, "llama2_7b", global_batch_size=64, sequence_length=4096, ks=[4])
    assert res is not None and len(res.stages) == 4 and [t["k"] for t in tried] == [4]
    out = export_config(res, "llama2_7b", 64, 4096, 32000, "bfloat16", "float32", str(tmp_path / "plan.json"))
    cfg = tc.parse_pipeline_config(str(tmp_path / "plan.json"))   # the trainer's reader accepts the planner's output
    assert cfg.world_size == 8 and cfg.latency == pytest.approx(res.latency_ms)
    assert all(len(s.gpu_ranks) == 2 for s in cfg.stages)


def test_bench_plans_are_valid_configs_and_deadlock_free():
    """bench.py's parallel plan for 1 / 2 / 4 / 8 GPUs parses as a training config (the named
    4 stages x 2-way ZeRO plan at 8) and its default schedule's p2p program completes under the
    serialised-process-group replay (checked on a 4-layer stand-in with the same stage graph)."""
    import importlib.util
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_main", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    from zorse_b200.config.training_config import parse_pipeline_dict
    from zorse_b200.parallel.p2p_sim import record_programs, simulate

    for n, stages, width in ((1, 1, 1), (2, 1, 2), (4, 2, 2), (8, 4, 2)):
        d, par = bench.build_config(n, "llama2_7b", 64, 1, 4096, 32000, "bfloat16", "1f1b")
        cfg = parse_pipeline_dict(d)
        assert len(cfg.stages) == stages and all(len(s.gpu_ranks) == width for s in cfg.stages)
        assert cfg.stages[-1].layer_partition[1] == 32 and cfg.num_microbatches == 64
        assert sorted(r for s in cfg.stages for r in s.gpu_ranks) == list(range(n))
        if stages > 1:
            small, _ = bench.build_config(n, "tiny_llama", 16, 1, 16, 128, "float32", "1f1b")
            small["autocast_dtype"] = "float32"
            assert simulate(record_programs(parse_pipeline_dict(small), "1f1b")) is None
    # the reference arm answers without touching a GPU
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"], capture_output=True,
                       text=True, timeout=120, cwd=root)
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert r.returncode == 0 and line["impl"] == "reference" and "unavailable" in line


def test_planner_lists_gpus_it_leaves_without_a_stage():
    """One fast GPU next to very slow ones on another machine: the slow group may get no layer;
    its ranks are then declared idle instead of silently missing from the config."""
    from zorse_b200.config.training_config import parse_pipeline_dict
    from zorse_b200.planner.plan import export_config, plan

    def gpu(rank, name, mem, machine, idx):
        return {"index": idx, "name": name, "memory_total_mib": mem, "id": f"gpu_{rank}", "machine": machine,
                "global_rank": rank}

    gl = [gpu(0, "p40", 23040, "m0", 0), gpu(1, "l4", 23034, "m0", 1), gpu(2, "b200", 183359, "m0", 2),
          gpu(3, "p40", 23040, "m1", 0)]
    data = {"machines": [{"machine": "m0", "num_gpus": 3, "gpus": gl[:3], "machine_index": 0},
                         {"machine": "m1", "num_gpus": 1, "gpus": gl[3:], "machine_index": 1}],
            "total_gpus": 4, "gpu_list": gl,
            "global_rank_map": {str(g["global_rank"]): {"machine": g["machine"], "local_rank": g["index"],
                                                        "machine_index": int(g["machine"][1])} for g in gl},
            "bandwidth": {"intranode_bandwidth": {"0": 25.0, "1": 25.0}, "intranode_latency": {"0": 1e-4, "1": 1e-4},
                          "internode_bandwidth": {"0": {"1": 1.0}, "1": {"0": 1.0}},
                          "internode_latency": {"0": {"1": 1e-3}, "1": {"0": 1e-3}}}}
    best, _ = plan(data, "opt_1b", global_batch_size=32, sequence_length=1024)
    d = export_config(best, "opt_1b", 32, 1024, 32000, "bfloat16", "float32", total_ranks=4)
    cfg = parse_pipeline_dict(d)
    assert cfg.world_size == 4
    named = {r for s in cfg.stages for r in s.gpu_ranks}
    assert named | set(cfg.unused_ranks) == {0, 1, 2, 3} and not (named & set(cfg.unused_ranks))


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 8), st.integers(1, 64), st.lists(st.floats(0.01, 100.0), min_size=8, max_size=8))
def test_shard_bounds_properties(R, blocks_per_rank, ratios):
    """Any positive ratios: offsets start at 0, end at n, are aligned, strictly increasing (every
    rank keeps at least one block), and equal ratios give equal shards."""
    from zorse_b200.engine.zero import shard_bounds
    from zorse_b200.models.layers import ALIGN

    n = R * blocks_per_rank * ALIGN
    b = shard_bounds(n, R, ratios[:R])
    assert b[0] == 0 and b[-1] == n and len(b) == R + 1
    assert all(x % ALIGN == 0 for x in b) and all(y > x for x, y in zip(b, b[1:]))
    assert shard_bounds(n, R, [1.0] * R) == shard_bounds(n, R)


def test_planner_with_tensor_parallel_lanes():
    """tp = 2 on eight GPUs: the plan numbers four lanes, the config carries tensor_parallel_size and names
    eight processes; lanes cost compute / 2 plus their collectives; mixed GPU models inside a lane are refused."""
    from zorse_b200.planner.plan import export_config, plan
    from zorse_b200.planner.tensor_parallel import coarsen, lane_collective_ms

    gl = [{"index": i, "name": "NVIDIA B200", "memory_total_mib": 183359, "id": f"gpu_{i}", "machine": "m0",
           "global_rank": i} for i in range(8)]
    data = {"machines": [{"machine": "m0", "num_gpus": 8, "machine_index": 0, "gpus": gl}], "gpu_list": gl,
            "total_gpus": 8, "bandwidth": {"internode_bandwidth": {}, "intranode_bandwidth": {"0": 770.0},
                                           "internode_latency": {}, "intranode_latency": {"0": 2e-5}}}
    lanes, members = coarsen(data, 2)
    assert lanes["total_gpus"] == 4 and members[1] == [2, 3] and lanes["gpu_list"][0]["memory_total_mib"] == 2 * 183359
    assert data["total_gpus"] == 8                                     # the input is left alone
    f, b = lane_collective_ms(data, [0, 1], 4096, 4096, 2)
    assert f > 0 and abs(b / f - 1.5) < 0.2                            # 6 against 4 collectives of the same size
    one, _ = plan(data, "llama2_7b", global_batch_size=64, sequence_length=4096, ks=[4])
    two, _ = plan(data, "llama2_7b", global_batch_size=64, sequence_length=4096, ks=[4], tensor_parallel_size=2)
    assert two is not None and len(two.stages) == 4 and all(len(s.gpu_ranks) == 1 for s in two.stages)
    d = export_config(two, "llama2_7b", 64, 4096, 32000, "bfloat16", "float32", total_ranks=4, tensor_parallel_size=2)
    cfg = tc.parse_pipeline_dict(d)
    assert cfg.tensor_parallel_size == 2 and cfg.world_size == 8 and cfg.num_lanes == 4
    assert one is not None and two.latency_ms != one.latency_ms
    mixed = [dict(g) for g in gl]
    mixed[1]["name"] = "NVIDIA H100"
    with pytest.raises(ValueError):
        coarsen(dict(data, gpu_list=mixed), 2)
    with pytest.raises(ValueError):
        coarsen(data, 3)


def test_leftover_layers_follow_the_reference_rule():
    # speeds 0.5 / 0.3 / 0.2 of 32 layers: exact 16 / 9.6 / 6.4, two layers left over
    t = [1 / 0.5, 1 / 0.3, 1 / 0.2]
    assert distribute_layers(32, t) == [17, 9, 6]                       # largest share first (reference)
    assert distribute_layers(32, t, rule="remainder") == [16, 10, 6]    # largest fractional remainder first


def test_fixed_plan_prediction_has_the_1f1b_and_gpipe_shapes():
    from zorse_b200.planner.predict import predict_step_ms

    def cfg(P, layers=32, M=64, R=2):
        per = layers // P
        return {"model_name": "llama2_7b", "global_batch_size": M, "microbatch_size": 1, "sequence_length": 4096,
                "vocab_size": 32000, "autocast_dtype": "bfloat16",
                "pipeline_config": [{"gpu_ranks": list(range(R * i, R * i + R)), "layer_partition": [i * per, (i + 1) * per],
                                     "num_microbatches_per_rank": [M // R] * R, "zero_config": [list(range(R * i, R * i + R))]}
                                    for i in range(P)]}

    table = {"llama2_7b": {"b200": {"4096": {"bfloat16": [[2.0, 0.0], [4.0, 0.0]]}}}}
    one = predict_step_ms(cfg(1, R=1), "1f1b", table=table)
    assert one["ramp_ms"] == 0 and abs(one["steady_ms"] - 64 * (32 * 6.0 + one["steady_ms"] / 64 - 32 * 6.0)) < 1e-6
    four = predict_step_ms(cfg(4), "1f1b", table=table)
    # ramps: the three stages that are not the bottleneck, one microbatch each; steady: 32 microbatches of the slowest
    assert 3 * 8 * 6.0 <= four["ramp_ms"] <= 3 * 8 * 6.0 + 2.0
    assert four["steady_ms"] >= 32 * 8 * 6.0
    deferred = predict_step_ms(cfg(4), "1f1b", table=table, defer_wgrad=True)
    assert deferred["ramp_ms"] < four["ramp_ms"] and deferred["steady_ms"] == four["steady_ms"]
    gp = predict_step_ms(cfg(4), "zero2", table=table)
    assert gp["recompute"] and gp["form"] == "gpipe" and gp["steady_ms"] > four["steady_ms"] * 1.25
    # layer-major on several stages: a stage passes microbatches on only from its last layer, so a stage starts
    # when its predecessor is in its last layer: with two stages of one layer each the passes pipeline perfectly,
    # with many layers per stage the stages run almost one after the other
    lm1 = predict_step_ms(cfg(2, layers=2, M=8, R=1), "layer_major", table=table)
    assert lm1["form"] == "layer_major"
    body = 8 * 2.0 + 2.0 + 8 * 6.0 + 6.0       # forward of 8 microbatches + one hand-over, backward with recompute likewise
    from zorse_b200.planner.latency import head_and_embedding_ms
    (hf, hb), (ef, eb) = head_and_embedding_ms("llama2_7b", "b200", 4096, 1, 32000)
    ends = 9 * (2 * hf + hb + 2 * ef + eb) + 1.0          # head and embedding (recomputed once) per microbatch, transfers
    assert body <= lm1["steady_ms"] + lm1["ramp_ms"] <= body + ends
    lm = predict_step_ms(cfg(4, M=64, R=1), "layer_major", table=table)
    serial = 32 * 64 * (2.0 + 6.0)               # every block on every microbatch, nothing overlapped
    assert 0.85 * serial < lm["steady_ms"] + lm["ramp_ms"] < 1.02 * serial
    assert predict_step_ms(cfg(1, R=1), "layer_major", table=table)["form"] == "gpipe"      # one stage: nothing to replay
    # a measured chain overhead scales the block times
    table["_chain_overhead"] = {"llama2_7b": {"b200": 1.1}}
    assert abs(predict_step_ms(cfg(4), "1f1b", table=table)["block_fwd_ms"] - 2.2) < 1e-9


def test_prediction_on_a_mixed_cluster_costs_every_rank_with_its_own_gpu():
    """`gpu` as a rank -> model mapping: a stage's single-microbatch time is its slowest rank's; its share of the
    steady state is the largest microbatches x time over its ranks, so giving the slow rank fewer microbatches helps
    exactly as far as it balances the products."""
    from zorse_b200.planner.predict import predict_step_ms

    table = {"llama2_7b": {"fast": {"4096": {"bfloat16": [[2.0, 0.0], [4.0, 0.0]]}},
                           "slow": {"4096": {"bfloat16": [[4.0, 0.0], [8.0, 0.0]]}}}}

    def cfg(counts):
        return {"model_name": "llama2_7b", "global_batch_size": sum(counts), "microbatch_size": 1, "sequence_length": 4096,
                "vocab_size": 32000, "autocast_dtype": "bfloat16",
                "pipeline_config": [{"gpu_ranks": [0, 1], "layer_partition": [0, 32], "num_microbatches_per_rank": counts,
                                     "zero_config": [[0, 1]]}]}

    same = predict_step_ms(cfg([12, 12]), "1f1b", table=table, gpu="fast")
    assert predict_step_ms(cfg([12, 12]), "1f1b", table=table, gpu={0: "fast", 1: "fast"})["ms"] == same["ms"]
    even = predict_step_ms(cfg([12, 12]), "1f1b", table=table, gpu={0: "fast", 1: "slow"})
    fair = predict_step_ms(cfg([16, 8]), "1f1b", table=table, gpu={0: "fast", 1: "slow"})
    over = predict_step_ms(cfg([20, 4]), "1f1b", table=table, gpu={0: "fast", 1: "slow"})
    assert even["block_fwd_ms"] == 4.0 and same["block_fwd_ms"] == 2.0
    t_fast, t_slow = same["stage_ms"][0], even["stage_ms"][0]        # one microbatch through the stage on either GPU
    assert t_slow - t_fast == pytest.approx(32 * 6.0)                # the blocks double, head and embedding do not change
    assert same["steady_ms"] == pytest.approx(12 * t_fast) and even["steady_ms"] == pytest.approx(12 * t_slow)
    assert fair["steady_ms"] == pytest.approx(max(16 * t_fast, 8 * t_slow)) and fair["steady_ms"] < even["steady_ms"]
    assert over["steady_ms"] == pytest.approx(20 * t_fast) and over["steady_ms"] > fair["steady_ms"]   # the fast rank is the long one now


def test_tail_deferral_rule_follows_the_drain_window():
    """The rule that picks how many layers of the last stage hold their weight gradients back: on by two layers for the
    4-stage plan with 32 microbatches per rank (measured: 1548 -> 1484 ms), off where the held-back work does not fit
    into the time the other stages drain, where little is gained, for recomputing schedules and for one stage."""
    from zorse_b200.planner.predict import best_tail_deferral, predict_step_ms

    def cfg(P, M, R, layers=32):
        per = layers // P
        return {"model_name": "llama2_7b", "global_batch_size": M, "microbatch_size": 1, "sequence_length": 4096,
                "vocab_size": 32000, "autocast_dtype": "bfloat16",
                "pipeline_config": [{"gpu_ranks": list(range(R * i, R * i + R)), "layer_partition": [i * per, (i + 1) * per],
                                     "num_microbatches_per_rank": [M // R] * R, "zero_config": [list(range(R * i, R * i + R))]}
                                    for i in range(P)]}

    assert best_tail_deferral(cfg(4, 64, 2), "1f1b") == 2
    assert best_tail_deferral(cfg(4, 32, 1), "1f1b") == 2
    assert best_tail_deferral(cfg(2, 64, 1), "1f1b") == 0            # 64 x 2 ms against a window of one stage's backward
    assert best_tail_deferral(cfg(2, 64, 2), "1f1b") == 0            # only the head would fit: under 1.5 % of the step
    assert best_tail_deferral(cfg(1, 64, 2), "1f1b") == 0
    assert best_tail_deferral(cfg(4, 64, 2), "zero2") == 0
    assert best_tail_deferral(cfg(4, 64, 2), "1f1b", max_hold_gib=4.0) == 0     # the held operands would not fit
    base = predict_step_ms(cfg(4, 64, 2), "1f1b")
    held = predict_step_ms(cfg(4, 64, 2), "1f1b", defer_tail_wgrad=2)
    assert held["tail_wgrad_ms"] == 0.0 and 0.03 < 1 - held["ms"] / base["ms"] < 0.05
    late = predict_step_ms(cfg(2, 64, 1), "1f1b", defer_tail_wgrad=2)
    assert late["tail_wgrad_ms"] > 50.0


def test_planner_cli_writes_schedule_and_tail_deferral(tmp_path):
    """`zorse_planner.py --schedule 1f1b` writes the schedule, this repository's prediction for it and the depth of the
    tail deferral into the file; the key survives a parse / to_dict round trip and reaches the schedule object."""
    import importlib.util
    import json
    import os

    from zorse_b200.config.training_config import parse_pipeline_config, parse_pipeline_dict, to_dict

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("planner_cli", os.path.join(root, "zorse_planner.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = tmp_path / "tc.json"
    rc = mod.main(["--cluster_info_file", os.path.join(root, "example", "cluster_info.json"), "--model_name", "llama2_7b",
                   "--global_batch_size", "64", "--sequence_length", "4096", "--num_stages", "4", "--microbatch_size", "1",
                   "--no_recompute", "--schedule", "1f1b", "--output", str(out)])
    assert rc == 0
    d = json.loads(out.read_text())
    assert d["schedule"] == "1f1b" and d["defer_tail_wgrad"] == 2 and 1400 < d["latency"] < 1650
    cfg = parse_pipeline_config(out)
    assert cfg.defer_tail_wgrad == 2 and to_dict(cfg)["defer_tail_wgrad"] == 2
    assert parse_pipeline_dict({k: v for k, v in d.items() if k != "defer_tail_wgrad"}).defer_tail_wgrad is None


def test_plan_ranks_candidates_by_the_schedule_the_trainer_will_run():
    """`plan(schedule=...)`: every candidate carries the stage-2 figure and the schedule-specific prediction; the
    winner is the one with the smallest schedule-specific prediction.  A cluster with two GPU models (no single
    profile row set) falls back to the stage-2 figure."""
    import json
    import os

    from zorse_b200.planner.cluster import load_cluster_info
    from zorse_b200.planner.plan import export_config, plan
    from zorse_b200.planner.predict import predict_step_ms

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    data = load_cluster_info(os.path.join(root, "example", "cluster_info.json"))
    kw = dict(global_batch_size=64, sequence_length=4096, microbatch_size=1, recompute=False)
    best, tried = plan(data, "llama2_7b", schedule="1f1b", **kw)
    assert all(t["schedule_ms"] is not None and t["latency_ms"] is not None for t in tried)
    win = min(tried, key=lambda t: t["schedule_ms"])
    assert len({tuple(s.gpu_ranks) for s in best.stages}) == win["k"]
    cfg = export_config(best, "llama2_7b", 64, 4096, 32000, "bfloat16", "float32")
    assert abs(predict_step_ms(cfg, "1f1b", recompute=False)["ms"] - win["schedule_ms"]) < 1e-6
    # layer-major on several stages runs them almost one after the other: the ranking must prefer few stages
    _, lm = plan(data, "llama2_7b", schedule="layer_major", global_batch_size=64, sequence_length=4096, microbatch_size=1)
    by_k = {t["k"]: t["schedule_ms"] for t in lm}
    assert by_k[1] < by_k[2] < by_k[4] < by_k[8]
    # a mixed cluster: every rank is costed with its own GPU model, so the plan with one slow GPU among its stages is
    # predicted slower than the all-B200 one
    mixed = json.loads(json.dumps(data))
    mixed["gpu_list"][0]["name"] = "NVIDIA H100 80GB HBM3"
    _, tr2 = plan(mixed, "llama2_7b", schedule="1f1b", ks=[8], **kw)
    _, tr1 = plan(data, "llama2_7b", schedule="1f1b", ks=[8], **kw)
    assert tr2[0]["schedule_ms"] > tr1[0]["schedule_ms"] * 1.05        # (the slow GPU's stage also gets fewer layers)


def test_drawings_of_the_gpu_graph_and_its_partition(tmp_path):
    import networkx as nx

    from zorse_b200.planner import visualize as V

    G = nx.Graph()
    for i in range(4):
        G.add_node(i, name="NVIDIA B200", machine=f"host{i // 2}", memory_total_mib=183359)
    for a, b, w in [(0, 1, 900.0), (2, 3, 900.0), (0, 2, 50.0), (1, 3, 50.0)]:
        G.add_edge(a, b, weight=w)
    parts = {0: 0, 1: 0, 2: 1, 3: 1}
    m = V.partition_metrics(G, parts)
    assert m["cut_weight"] == 100.0 and m["internal_weight"] == 1800.0 and m["balance"] == 1.0
    assert m["partition_sizes"] == {0: 2, 1: 2} and abs(m["ratio_cut_to_total"] - 100 / 1900) < 1e-12
    sc = V.scene_partitioned(G, parts)
    assert sorted(e["dashed"] for e in sc.edges) == [False, False, True, True]
    assert {n["color"] for n in sc.nodes if parts[n["id"]] == 0} != {n["color"] for n in sc.nodes if parts[n["id"]] == 1}
    assert all(0.0 <= n["x"] <= 1.0 and 0.0 <= n["y"] <= 1.0 for n in sc.nodes)
    sm = V.scene_with_metrics(G, parts)
    assert any("Cut value: 100.00" in ln for ln in sm.side_text) and any("P1: 2 nodes" in ln for ln in sm.side_text)
    g = V.scene_graph(G)
    assert len(g.legend) == 2 and g.nodes[0]["label"].startswith("B200\n179.1GB")
    out = V.visualize_partitions_with_metrics(G, parts, output_file=str(tmp_path / "p.svg"))
    txt = open(out).read()
    assert txt.startswith("<svg") and "stroke-dasharray" in txt and "Balance: 1.00" in txt
    assert V.visualize_partition(G, parts, str(tmp_path / "plan.svg"))
    assert (tmp_path / "plan_graph.svg").exists() and (tmp_path / "plan_partitioned.svg").exists()


def test_latency_driven_microbatch_routing():
    """Ranks of unequal speed: the first stage hands its microbatches on in the order they finish, the next stage
    feeds the rank with most work ahead first (reference zorse_utils/pipeline_comm.py:193-303); equal ranks reduce to
    round-robin; the plan stays a valid many-to-many routing and the 1F1B order built on it completes."""
    from zorse_b200.parallel.p2p_plan import create_static_comm_plans, latency_owners, plan_1f1b_order
    from zorse_b200.parallel.p2p_sim import preflight

    assert latency_owners([2, 2], [1.0, 1.0], receiver=False) == [0, 1, 0, 1]
    assert latency_owners([2, 2], [1.0, 1.0], receiver=True) == [1, 0, 1, 0]
    # a rank twice as fast with three times the microbatches: it finishes 0, 1, 2 at t = 0, 1, 2; the slow one at 0
    assert latency_owners([3, 1], [1.0, 2.0], receiver=False) == [1, 0, 0, 0]
    # receiving side: work ahead 3, 2, 1 (fast rank) and 2 (slow rank): fast, then the tie goes to the slower rank
    assert latency_owners([3, 1], [1.0, 2.0], receiver=True) == [0, 1, 0, 0]
    d = {"model_name": "tiny_llama", "global_batch_size": 8, "microbatch_size": 1, "sequence_length": 64,
         "comm_plan": "latency", "rank_latency_ms": {"0": 1.0, "1": 2.0, "2": 1.5, "3": 1.5},
         "pipeline_config": [
             {"gpu_ranks": [0, 1], "num_microbatches_per_rank": [6, 2], "layer_partition": [0, 2], "zero_config": [[0, 1]]},
             {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [4, 4], "layer_partition": [2, 4], "zero_config": [[2, 3]]}]}
    cfg = tc.parse_pipeline_dict(d)
    assert cfg.comm_plan == "latency" and cfg.rank_latency_ms[1] == 2.0
    assert tc.to_dict(cfg)["rank_latency_ms"] == {"0": 1.0, "1": 2.0, "2": 1.5, "3": 1.5}
    plans = create_static_comm_plans(cfg)            # validates mirror-image sends / receives and counts
    assert len(plans[0].stages[0].microbatches) == 6 and len(plans[1].stages[0].microbatches) == 2
    # per microbatch rank 0 needs 2 ms (2 layers x 1.0), rank 1 needs 4 ms: completions at 0, 2, 4, 6, 8, 10 and 0, 4;
    # ties go to the slower rank first (the reference sorts (time, -latency, rank) tuples)
    assert plans[0].stages[0].microbatches == [1, 2, 4, 5, 6, 7] and plans[1].stages[0].microbatches == [0, 3]
    base = tc.parse_pipeline_dict({k: v for k, v in d.items() if k not in ("comm_plan", "rank_latency_ms")})
    assert create_static_comm_plans(base)[1].stages[0].microbatches == [2, 6]          # by counts alone
    order = plan_1f1b_order(cfg)
    assert sorted(op for op, _ in order[1]) == ["B", "B", "F", "F"]
    for sched in ("layer_major", "zero2", "1f1b"):
        assert preflight(cfg, sched) is None, sched      # the p2p program of every schedule completes under NCCL's rules


@pytest.mark.parametrize("n,want", [(1, ("1f1b", "library", 0, 1)), (2, ("1f1b", "fused", 0, 1)),
                                    (4, ("1f1b", "fused", 0, 2)), (8, ("1f1b", "fused", 2, 4))])
def test_bench_defaults_per_gpu_count(n, want, monkeypatch):
    """What `bench.py --gpus N` hands to the trainer with no other flag: 1F1B, this repository's fused collectives from
    two GPUs up, and the tail deferral the planner's rule picks (two layers on the 4-stage plan only)."""
    import importlib.util
    import os
    import sys

    import zorse_b200.trainer as trainer_mod

    class Captured(Exception):
        pass

    def fake_trainer(cfg, opt):
        raise Captured((cfg, opt))

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_script_defaults", os.path.join(root, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    monkeypatch.setattr(trainer_mod, "Trainer", fake_trainer)
    monkeypatch.setenv("WORLD_SIZE", str(n))
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", str(n)])
    with pytest.raises(Captured) as e:
        mod.main()
    cfg, opt = e.value.args[0]
    assert (opt.schedule, opt.collectives, opt.defer_tail_wgrad, len(cfg.stages)) == want
    assert opt.activation_recompute is None and not opt.defer_wgrad and not opt.prepost_recv
    assert cfg.model_name == "llama2_7b" and cfg.global_batch_size == 64 and cfg.sequence_length == 4096
