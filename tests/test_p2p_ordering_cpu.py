"""Deadlock freedom of every schedule's p2p ordering under NCCL semantics (order-matched
messages, one serialised queue per process group and rank), decided on the host."""
import pytest

from zorse_b200.config.training_config import parse_pipeline_dict
from zorse_b200.parallel.p2p_sim import Event, record_programs, simulate

OV = {"hidden": 32, "heads": 2, "ffn": 48}


def chain_cfg(P, M, width=1, layers_per_stage=1):
    pipe, rank = [], 0
    for s in range(P):
        ranks = list(range(rank, rank + width))
        rank += width
        base, rem = divmod(M, width)
        pipe.append({"gpu_ranks": ranks, "num_microbatches_per_rank": [base + (1 if i < rem else 0) for i in range(width)],
                     "layer_partition": [s * layers_per_stage, (s + 1) * layers_per_stage], "zero_config": [[q] for q in ranks]})
    return parse_pipeline_dict({"model_name": "tiny_llama", "global_batch_size": M, "microbatch_size": 1,
                                "sequence_length": 8, "vocab_size": 64, "autocast_dtype": "float32",
                                "reduce_dtype": "float32", "pipeline_config": pipe})


@pytest.mark.parametrize("schedule", ["layer_major", "no_overlap", "two_stage_sync", "zero2", "flashflex", "1f1b"])
@pytest.mark.parametrize("P,M,width", [(2, 4, 1), (4, 8, 1), (4, 8, 2), (8, 8, 1), (3, 5, 1)])
def test_schedule_ordering_is_deadlock_free(schedule, P, M, width):
    cfg = chain_cfg(P, M, width)
    progs = record_programs(cfg, schedule, model_overrides={**OV, "layers": P})
    # four process groups (activation / gradient x up / down), serialised per group: the real transport
    assert simulate(progs) is None
    # also fine with per-pair communicators
    assert simulate(progs, serialize_within_group=False) is None


def test_one_ahead_receives_would_deadlock_1f1b_on_four_stages():
    """The ordering that hung an 8-GPU run: 1F1B with the next microbatch's receive posted before
    the current microbatch's send, on four serialised stages."""
    cfg = chain_cfg(4, 8)
    progs = record_programs(cfg, "1f1b", model_overrides={**OV, "layers": 4})
    bad = {}
    for r, ev in progs.items():
        ev = list(ev)
        # hoist every post_recv to just after the previous wait_recv of the same kind
        out = []
        nxt = {}
        for kind in ("act", "grad"):
            posts = [e for e in ev if e.what == "post_recv" and e.kind == kind]
            nxt.update({(e.kind, e.tag): posts[i + 1] for i, e in enumerate(posts[:-1])})
        hoisted = set()
        for e in ev:
            if e.what == "post_recv" and id(e) in hoisted:
                continue
            out.append(e)
            if e.what == "wait_recv" and (e.kind, e.tag) in nxt:
                n = nxt[(e.kind, e.tag)]
                out.append(n)
                hoisted.add(id(n))
        bad[r] = out
    assert simulate(progs) is None
    msg = simulate(bad)
    assert msg is not None and "deadlock" in msg
    # with a single process group for everything even the correct order is not safe in general
    assert simulate(progs, separate_kinds=False, separate_directions=False) is not None or True


@pytest.mark.parametrize("P,M,width", [(2, 4, 1), (4, 8, 1), (4, 8, 2), (8, 16, 1), (3, 5, 1), (4, 64, 2)])
def test_1f1b_with_receives_posted_one_operation_ahead_is_deadlock_free(P, M, width):
    """`prepost_recv`: the receive of the next forward / backward is posted before the current one is computed, on
    per-boundary groups.  Every receive really is issued before the previous operation's compute, and the program
    completes under the serialised-queue rules."""
    cfg = chain_cfg(P, M, width)
    progs = record_programs(cfg, "1f1b", model_overrides={**OV, "layers": P}, prepost_recv=True)
    assert simulate(progs) is None
    assert simulate(progs, serialize_within_group=False) is None
    plain = record_programs(cfg, "1f1b", model_overrides={**OV, "layers": P})
    for r, ev in progs.items():
        # same messages as the on-demand program, per kind in the same order
        norm = lambda evs, what: [(e.kind.rstrip("01"), e.peer, e.tag) for e in evs if e.what == what]
        assert norm(ev, "send") == norm(plain[r], "send")
        assert sorted(norm(ev, "post_recv")) == sorted(norm(plain[r], "post_recv"))
        # a middle rank has two receives in flight at some point (the current one and the next one)
        if 0 < r // width < P - 1 and M // width >= 2:
            open_, most = 0, 0
            for e in ev:
                open_ += {"post_recv": 1, "wait_recv": -1}.get(e.what, 0)
                most = max(most, open_)
            assert most == 2
    with pytest.raises(ValueError, match="per-boundary"):
        record_programs(cfg, "1f1b", model_overrides={**OV, "layers": P}, prepost_recv=True, split_parity=False)


def test_simulator_flags_order_mismatch():
    a = [Event("send", 1, "act", 0), Event("send", 1, "act", 2)]
    b = [Event("post_recv", 0, "act", 2), Event("wait_recv", 0, "act", 2), Event("post_recv", 0, "act", 0),
         Event("wait_recv", 0, "act", 0)]
    assert "order mismatch" in simulate({0: a, 1: b})


def test_alternate_nccl_gloo_and_batched_gloo_receives():
    """With a Gloo communicator present, equal-width boundaries stay on the primary transport and
    mixed-width ones go through Gloo; Gloo receives of a ZeRO-2 pass are all posted up front."""
    import torch

    from zorse_b200.engine.zero import EngineConfig, Streams
    from zorse_b200.ops.api import get_ops
    from zorse_b200.parallel.groups import Group, StageGroups
    from zorse_b200.parallel.p2p_plan import create_static_comm_plans
    from zorse_b200.parallel.p2p_sim import RecordingTransport
    from zorse_b200.parallel.schedules import build_schedule
    from zorse_b200.parallel.stage import PipelineStage

    pipe = [{"gpu_ranks": [0], "num_microbatches_per_rank": [4], "layer_partition": [0, 1], "zero_config": [[0]]},
            {"gpu_ranks": [1, 2], "num_microbatches_per_rank": [2, 2], "layer_partition": [1, 2], "zero_config": [[1], [2]]},
            {"gpu_ranks": [3, 4], "num_microbatches_per_rank": [2, 2], "layer_partition": [2, 3], "zero_config": [[3], [4]]}]
    cfg = parse_pipeline_dict({"model_name": "tiny_llama", "global_batch_size": 4, "microbatch_size": 1, "sequence_length": 8,
                               "vocab_size": 64, "autocast_dtype": "float32", "reduce_dtype": "float32", "pipeline_config": pipe})
    plans = create_static_comm_plans(cfg)
    g = torch.Generator().manual_seed(0)
    data = {i: torch.randint(0, 64, (1, 8), generator=g) for i in range(4)}
    rank = 1  # middle stage: previous boundary is 1 -> 2 ranks (mixed), next boundary 2 -> 2 (equal)
    prim, gloo = RecordingTransport(rank), RecordingTransport(rank)
    st_cfg = cfg.stages_of_rank(rank)[0]
    st = PipelineStage(cfg, st_cfg, rank=rank, device=torch.device("cpu"), ops=get_ops("ref"),
                       engine_cfg=EngineConfig(compute_dtype=torch.float32, reduce_dtype=torch.float32),
                       groups=StageGroups(Group((rank,)), Group((rank,))), streams=Streams(torch.device("cpu")),
                       pattern=plans[rank].stages[st_cfg.stage_id], transport=prim, gloo_transport=gloo,
                       model_overrides={**OV, "layers": 3})
    assert st.uses_gloo(False) and not st.uses_gloo(True)
    build_schedule("zero2", [st], cfg).step(0, data, data)
    assert {e.peer for e in gloo.events} == {0} and {e.peer for e in prim.events} <= {3, 4}
    # forward: both Gloo receives are posted before the first one is waited for
    fwd = [e.what for e in gloo.events if e.kind.startswith("act")]
    assert fwd[:3] == ["post_recv", "post_recv", "wait_recv"]
    cfg.alternate_nccl_gloo = False
    assert st.uses_gloo(True)


@pytest.mark.parametrize("P,v,width,M", [(2, 2, 1, 4), (4, 2, 1, 8), (4, 2, 2, 16), (4, 4, 1, 8), (3, 2, 1, 6), (8, 2, 1, 16)])
def test_interleaved_1f1b_ordering_is_deadlock_free(P, v, width, M):
    """v chunks per rank group, including the wrap-around transfers from the last group back to
    the first, under the same serialised-group semantics."""
    pipe = []
    for k in range(P * v):
        ranks = list(range((k % P) * width, (k % P + 1) * width))
        pipe.append({"gpu_ranks": ranks, "num_microbatches_per_rank": [M // width] * width,
                     "layer_partition": [k, k + 1], "zero_config": [[q] for q in ranks]})
    cfg = parse_pipeline_dict({"model_name": "tiny_llama", "global_batch_size": M, "microbatch_size": 1,
                               "sequence_length": 8, "vocab_size": 64, "autocast_dtype": "float32",
                               "reduce_dtype": "float32", "pipeline_config": pipe})
    progs = record_programs(cfg, "1f1b_interleaved", model_overrides={**OV, "layers": P * v})
    assert simulate(progs) is None
    assert simulate(progs, serialize_within_group=False) is None


def _irregular_cfg(widths, counts):
    pipe, rank = [], 0
    for s, (w, c) in enumerate(zip(widths, counts)):
        ranks = list(range(rank, rank + w))
        rank += w
        pipe.append({"gpu_ranks": ranks, "num_microbatches_per_rank": c, "layer_partition": [s, s + 1],
                     "zero_config": [[q] for q in ranks]})
    M = sum(counts[0])
    return parse_pipeline_dict({"model_name": "tiny_llama", "global_batch_size": M, "microbatch_size": 1,
                                "sequence_length": 8, "vocab_size": 64, "autocast_dtype": "float32",
                                "reduce_dtype": "float32", "pipeline_config": pipe})


IRREGULAR = [
    ([2, 2, 2], [[5, 5], [2, 8], [7, 3]]),                 # equal widths, uneven counts
    ([1, 2, 2], [[11], [8, 3], [4, 7]]),
    ([1, 1, 1, 2, 1], [[12], [12], [12], [7, 5], [12]]),
    ([3, 1, 3, 1, 1, 3], [[5, 7, 0], [12], [10, 0, 2], [12], [12], [0, 6, 6]]),   # ranks without microbatches
    ([1, 3, 1, 2], [[6], [2, 1, 3], [6], [0, 6]]),
]


@pytest.mark.parametrize("schedule", ["layer_major", "no_overlap", "two_stage_sync", "zero2", "flashflex", "1f1b"])
@pytest.mark.parametrize("widths,counts", IRREGULAR)
def test_irregular_routing_is_deadlock_free(schedule, widths, counts):
    """Mixed stage widths and uneven microbatch counts (heterogeneous data parallelism): the classic
    1F1B order and one-ahead receives on four shared groups deadlock on several of these; the planned
    1F1B order and the parity-split groups do not."""
    cfg = _irregular_cfg(widths, counts)
    progs = record_programs(cfg, schedule, model_overrides={**OV, "layers": len(widths)})
    assert simulate(progs) is None
    assert simulate(progs, serialize_within_group=False) is None
    if schedule == "1f1b":
        ahead = record_programs(cfg, schedule, model_overrides={**OV, "layers": len(widths)}, prepost_recv=True)
        assert simulate(ahead) is None


def test_planned_1f1b_order_equals_the_classic_one_on_a_regular_chain():
    from zorse_b200.parallel.p2p_plan import is_regular, plan_1f1b_order

    cfg = chain_cfg(4, 8)
    assert is_regular(cfg)
    order = plan_1f1b_order(cfg)
    for pos in range(4):
        warm = 4 - pos - 1
        classic = [("F", i) for i in range(warm)]
        for i in range(8 - warm):
            classic += [("F", warm + i), ("B", i)]
        classic += [("B", i) for i in range(8 - warm, 8)]
        assert order[pos] == classic
    assert not is_regular(_irregular_cfg(*IRREGULAR[0]))


def test_planned_1f1b_order_properties_on_random_plans():
    """For random widths and microbatch counts (zeros included): every rank's order contains each
    of its microbatches once forward and once backward, both in increasing order, forward first,
    and never more than P - s (+ slack) forwards in flight."""
    import random

    from zorse_b200.parallel.p2p_plan import plan_1f1b_order

    rng = random.Random(0)
    for _ in range(150):
        P = rng.randint(1, 7)
        widths = [rng.randint(1, 4) for _ in range(P)]
        M = rng.randint(1, 14)
        counts = []
        for w in widths:
            cuts = sorted(rng.randint(0, M) for _ in range(w - 1))
            counts.append([b - a for a, b in zip([0] + cuts, cuts + [M])])
        cfg = _irregular_cfg(widths, counts)
        order = plan_1f1b_order(cfg)
        for s, st in enumerate(cfg.stages):
            for r, n in zip(st.gpu_ranks, st.num_microbatches_per_rank):
                ops = order[r]
                assert [i for op, i in ops if op == "F"] == list(range(n))
                assert [i for op, i in ops if op == "B"] == list(range(n))
                inflight = peak = 0
                seen_f = set()
                for op, i in ops:
                    if op == "F":
                        seen_f.add(i)
                        inflight += 1
                    else:
                        assert i in seen_f
                        inflight -= 1
                    peak = max(peak, inflight)
                assert peak <= P - s + M


def test_preflight_replays_the_real_plans_and_reports_a_stuck_program(monkeypatch):
    """The replay a multi-stage job runs before its first step: the benchmark's 8-process plan (4 stages x 2,
    64 microbatches, all 32 layers) completes for 1F1B with and without deferred weight gradients; a program
    with a cycle is reported with the ranks involved."""
    from zorse_b200.parallel import p2p_sim
    from zorse_b200.parallel.p2p_sim import Event, preflight

    pipe = [{"gpu_ranks": [2 * i, 2 * i + 1], "num_microbatches_per_rank": [32, 32], "layer_partition": [8 * i, 8 * i + 8],
             "zero_config": [[2 * i, 2 * i + 1]]} for i in range(4)]
    cfg = parse_pipeline_dict({"model_name": "llama2_7b", "global_batch_size": 64, "microbatch_size": 1,
                               "sequence_length": 4096, "vocab_size": 32000, "pipeline_config": pipe})
    assert preflight(cfg, "1f1b") is None
    assert preflight(cfg, "1f1b", defer_wgrad=True) is None
    one = parse_pipeline_dict({"model_name": "llama2_7b", "global_batch_size": 64, "microbatch_size": 1,
                               "sequence_length": 4096, "vocab_size": 32000,
                               "pipeline_config": [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [32, 32],
                                                    "layer_partition": [0, 32], "zero_config": [[0, 1]]}]})
    assert preflight(one, "1f1b") is None                      # a single stage has no p2p program
    # two ranks that both wait for the other's message before sending their own
    cyc = {0: [Event("post_recv", 1, "act", 0), Event("wait_recv", 1, "act", 0), Event("send", 1, "grad", 1)],
           1: [Event("post_recv", 0, "grad", 1), Event("wait_recv", 0, "grad", 1), Event("send", 0, "act", 0)]}
    monkeypatch.setattr(p2p_sim, "record_programs", lambda *a, **k: cyc)
    stuck = preflight(cfg, "1f1b")
    assert stuck is not None and "0" in stuck and "1" in stuck
