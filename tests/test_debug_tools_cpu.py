"""Debug aids: stream-order checker (vector clocks), deterministic replay, named ranges."""
import pytest
import torch

from zorse_b200.utils import ranges
from zorse_b200.utils.stream_check import StreamOrderChecker, StreamOrderError


def test_read_after_event_wait_is_ordered():
    c = StreamOrderChecker()
    c.wrote("full", "comm")
    c.record("ev", "comm")
    assert not c.read("full", "compute", "before the wait")       # the race
    c.wait_event("compute", "ev")
    assert c.read("full", "compute", "after the wait")
    assert len(c.violations) == 1 and "comm" in str(c.violations[0])


def test_event_recorded_before_the_write_does_not_cover_it():
    c = StreamOrderChecker()
    c.record("early", "comm")
    c.wrote("grad", "comm")
    c.wait_event("compute", "early")
    assert not c.read("grad", "compute")


def test_ordering_is_transitive_and_same_stream_is_free():
    c = StreamOrderChecker()
    c.wrote("act", "compute")
    assert c.read("act", "compute")                 # program order on one stream
    c.wait_stream("copy", "compute")                # copy stream waits for compute ...
    c.wrote("host", "copy")
    c.record("done", "copy")
    c.wait_event("other", "done")                   # ... a third stream waits for the copy
    assert c.read("host", "other") and c.read("act", "other")


def test_missing_wait_stream_is_the_reference_bug_class():
    """Activation copied to the host on a side stream that never waited for the compute stream."""
    c = StreamOrderChecker(strict=True)
    c.wrote(("stash_src", 1), "compute")
    with pytest.raises(StreamOrderError, match="without having waited"):
        c.read(("stash_src", 1), "copy", "D2H copy")
    c.wait_stream("copy", "compute")
    assert c.read(("stash_src", 1), "copy")


def test_host_synchronize_orders_everything():
    c = StreamOrderChecker()
    c.wrote("x", "comm")
    c._clock("compute")
    c.synchronize()
    assert c.read("x", "compute")
    assert "no violation" in c.report()


def test_module_hooks_are_noops_when_inactive():
    from zorse_b200.utils import stream_check as SC

    assert SC.active() is None
    SC.wrote("k", "s")          # must not touch torch.cuda on a CPU box
    SC.read("k", "s")


def _tiny_trainer():
    from zorse_b200.config.training_config import parse_pipeline_dict
    from zorse_b200.trainer import Trainer, TrainerOptions

    cfg = parse_pipeline_dict({
        "model_name": "tiny_llama", "global_batch_size": 4, "microbatch_size": 2, "sequence_length": 16,
        "vocab_size": 128, "autocast_dtype": "float32", "reduce_dtype": "float32",
        "pipeline_config": [{"gpu_ranks": [0], "num_microbatches_per_rank": [2], "layer_partition": [0, 4],
                             "zero_config": [[0]]}]})
    tr = Trainer(cfg, TrainerOptions(schedule="layer_major", ops="ref"))
    batch = tr.synthetic_batch()
    inputs, targets, _ = tr.to_device(batch)
    return tr, inputs, targets


def test_replay_is_bit_identical_on_the_oracle_backend():
    from zorse_b200.utils.replay import replay_check

    tr, inputs, targets = _tiny_trainer()
    rep = replay_check(tr, inputs, targets)
    assert rep["identical"] and rep["differing_units"] == [] and rep["loss"][0] == rep["loss"][1]
    assert tr.step_idx == 1


def test_replay_reports_the_unit_that_differs():
    from zorse_b200.utils.replay import replay_check

    tr, inputs, targets = _tiny_trainer()
    orig = tr.ops.adam_step
    calls = {"n": 0}

    def noisy(master, *a, **kw):
        orig(master, *a, **kw)
        calls["n"] += 1
        if calls["n"] == len(tr.stages[0].engine.units) + 2:     # second unit of the second run
            master.add_(1e-3)

    tr.ops.adam_step = noisy
    rep = replay_check(tr, inputs, targets, tolerance=1e-6)
    assert not rep["identical"] and not rep["within_tolerance"]
    assert len(rep["differing_units"]) == 1 and rep["differing_units"][0]["max_abs_diff"] > 5e-4


def test_ranges_name_every_engine_phase():
    tr, inputs, targets = _tiny_trainer()
    log: list = []
    ranges.enable(True)
    ranges.capture(log)
    try:
        tr.train_step(inputs, targets)
    finally:
        ranges.capture(None)
        ranges.enable(False)
    seen = set(log)
    assert {"fwd.embedding", "fwd.block", "fwd.head", "bwd.block", "bwd.head", "recompute.block"} <= seen
    assert ranges.phase("x").__class__.__name__ == "_Null"


def test_shift_labels_training_matches_autograd():
    """Next-token targets with an ignored last position: loss and gradients of the explicit
    backward equal autograd's (ignored rows contribute zero loss and zero gradient)."""
    from zorse_b200.config.training_config import parse_pipeline_dict
    from zorse_b200.trainer import Trainer, TrainerOptions
    from zorse_b200.utils.oracle import OracleTrainer

    d = {"model_name": "tiny_llama", "global_batch_size": 4, "microbatch_size": 2, "sequence_length": 16,
         "vocab_size": 128, "autocast_dtype": "float32", "reduce_dtype": "float32",
         "pipeline_config": [{"gpu_ranks": [0], "num_microbatches_per_rank": [2], "layer_partition": [0, 4],
                              "zero_config": [[0]]}]}
    cfg = parse_pipeline_dict(d)
    tr = Trainer(cfg, TrainerOptions(schedule="layer_major", ops="ref", shift_labels=True))
    batch = tr.synthetic_batch()
    assert torch.equal(batch["targets"][..., :-1], batch["inputs"][..., 1:]) and (batch["targets"][..., -1] == -100).all()
    orc = OracleTrainer(cfg)
    want = [orc.step(batch) for _ in range(2)]
    got = [tr.train_step_from_host(batch) for _ in range(2)]
    assert all(abs(a - b) < 2e-4 for a, b in zip(got, want)), (got, want)
    for u, f in zip(tr.stages[0].engine.units, orc.flats):
        assert (u.full_master()[: f.numel()] - f.detach()).abs().max() < 5e-4


def test_canary_detects_writes_outside_a_guarded_buffer():
    from zorse_b200.utils import canary

    canary.reset()
    alloc = lambda k, dt: torch.zeros(k, dtype=dt)
    assert canary.guarded(10, torch.float32, alloc, "plain").numel() == 10      # off: plain allocation
    buf = canary.guarded(100, torch.bfloat16, alloc, "unit 3 gradients", force=True)
    assert buf.numel() == 100 and buf.data_ptr() % 16 == 0
    buf.fill_(1.0)                              # writes inside the payload are fine
    assert canary.check_all() == []
    raw = buf._base
    raw[canary.guard_elems(torch.bfloat16) + 100] = 7.0      # first element after the payload
    assert canary.check_all(raise_on_error=False) == ["unit 3 gradients (band after the buffer)"]
    with pytest.raises(canary.CanaryError, match="unit 3 gradients"):
        canary.check_all()
    canary.reset()


def test_deferred_wgrad_front_queues_in_order_and_passes_everything_else_through():
    from zorse_b200.parallel.stage import DeferredWgrad

    calls = []

    class Ops:
        name = "fake"

        def linear_wgrad(self, *a, **k):
            calls.append(("wgrad", a, k))

        def linear_dgrad(self, *a):
            calls.append(("dgrad", a))
            return "dx"

    d = DeferredWgrad(Ops())
    assert d.name == "fake" and d.linear_dgrad(1) == "dx"
    d.linear_wgrad(1, 2, accumulate=True)                 # not active: runs at once
    assert calls == [("dgrad", (1,)), ("wgrad", (1, 2), {"accumulate": True})]
    d.active = True
    d.linear_wgrad("a")
    d.linear_dgrad(2)
    d.linear_wgrad("b")
    assert [c[0] for c in calls] == ["dgrad", "wgrad", "dgrad"]     # the two weight gradients are held back
    d.active = False
    d.flush()
    assert [c[1][0] for c in calls[3:]] == ["a", "b"]               # in the order they were asked for
    d.flush()
    assert len(calls) == 5
