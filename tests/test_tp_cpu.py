"""Tensor parallelism with sequence-parallel activations on CPU ranks (gloo): every combination with
pipeline stages and ZeRO data parallelism must reproduce the single-process oracle (same loss, same
parameters after two steps, once the slices are put back together)."""
import pytest
import torch

from dist_utils import run_workers
from test_dist_cpu import _oracle, tiny_cfg
from zorse_b200.config.training_config import ConfigError, parse_pipeline_dict, to_dict


def _worker(rank, world, cfg_dict, opts, steps):
    from zorse_b200.trainer import Trainer, TrainerOptions

    cfg = parse_pipeline_dict(cfg_dict)
    tr = Trainer(cfg, TrainerOptions(backend="gloo", **opts))
    batch = tr.synthetic_batch()
    losses = [tr.global_loss(tr.train_step_from_host(batch)) for _ in range(steps)]
    params = {u.gid: u.full_master()[: u.layer.layout()[1]].clone() for st in tr.stages for u in st.engine.units}
    return {"losses": losses, "params": params, "tp_index": tr.tp_index, "lane": tr.lane,
            "all_reduces": [c.all_reduces for c in tr.counters()]}


def _check_tp(results, cfg_dict, steps=2, ptol=5e-4):
    from zorse_b200.models import registry

    cfg = parse_pipeline_dict(cfg_dict)
    tp = cfg.tensor_parallel_size
    spec = registry.get_spec(cfg.model_name, vocab=cfg.vocab_size)
    want_losses, want_params = _oracle(cfg_dict, steps)
    for res in results:
        for a, b in zip(res["losses"], want_losses):
            assert abs(a - b) < 2e-4, (res["losses"], want_losses)
    # put the slices of every block back together, lane by lane
    lanes = sorted({r["lane"] for r in results})
    for lane in lanes:
        mine = sorted((r for r in results if r["lane"] == lane), key=lambda r: r["tp_index"])
        assert [r["tp_index"] for r in mine] == list(range(tp))
        for gid in mine[0]["params"]:
            if 1 <= gid <= spec.layers:
                whole = torch.zeros_like(want_params[gid])
                for r in mine:
                    registry.make_block(spec, tp, r["tp_index"]).store_into_whole(r["params"][gid], whole)
                got = [whole]
            else:
                got = [r["params"][gid] for r in mine]     # embedding / head: every process holds all of it
            for g in got:
                err = (g - want_params[gid][: g.numel()]).abs().max().item()
                assert err < ptol, f"lane {lane} unit {gid}: max param error {err}"


ONE_LANE = [{"gpu_ranks": [0], "num_microbatches_per_rank": [4], "layer_partition": [0, 4], "zero_config": [[0]]}]
TWO_STAGES = [{"gpu_ranks": [0], "num_microbatches_per_rank": [4], "layer_partition": [0, 2], "zero_config": [[0]]},
              {"gpu_ranks": [1], "num_microbatches_per_rank": [4], "layer_partition": [2, 4], "zero_config": [[1]]}]
TWO_DP = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [2, 2], "layer_partition": [0, 4], "zero_config": [[0, 1]]}]


@pytest.mark.parametrize("schedule,recompute", [("layer_major", None), ("1f1b", False)])
def test_tp2_one_lane(schedule, recompute):
    cfg = tiny_cfg(ONE_LANE, tensor_parallel_size=2)
    res = run_workers(2, _worker, cfg, {"schedule": schedule, "activation_recompute": recompute}, 2)
    _check_tp(res, cfg)
    assert all(n > 0 for r in res for n in r["all_reduces"])      # norm / embedding / head gradients summed over the lane


@pytest.mark.parametrize("schedule", ["1f1b"])
def test_tp2_two_stages(schedule):
    """2 stages x tp 2 = 4 processes; process l*2+t sends its rows to process (l+1)*2+t."""
    cfg = tiny_cfg(TWO_STAGES, tensor_parallel_size=2)
    res = run_workers(4, _worker, cfg, {"schedule": schedule}, 2)
    _check_tp(res, cfg)


@pytest.mark.parametrize("schedule,oib", [("zero2", True)])
def test_tp2_two_way_zero(schedule, oib):
    """ZeRO shard groups connect the processes that hold the same slice: {0, 2} and {1, 3}."""
    cfg = tiny_cfg(TWO_DP, tensor_parallel_size=2)
    res = run_workers(4, _worker, cfg, {"schedule": schedule, "optimizer_in_backward": oib}, 2)
    _check_tp(res, cfg)


def test_tp_config_round_trip_and_errors():
    cfg = parse_pipeline_dict(tiny_cfg(TWO_STAGES, tensor_parallel_size=4))
    assert cfg.num_lanes == 2 and cfg.world_size == 8
    assert to_dict(cfg)["tensor_parallel_size"] == 4
    assert "tensor_parallel_size" not in to_dict(parse_pipeline_dict(tiny_cfg(TWO_STAGES)))
    with pytest.raises(ConfigError):
        parse_pipeline_dict(tiny_cfg(TWO_STAGES, tensor_parallel_size=0))


def test_slices_tile_the_unsplit_block():
    """take_slice / put_slice are inverse, the slices of all processes cover every parameter exactly once,
    and replicated parameters are the ones reported for the lane-wide gradient sum."""
    from zorse_b200.models import registry

    spec = registry.get_spec("tiny_llama", vocab=512)
    whole = registry.make_block(spec)
    _, n = whole.layout()
    ref = torch.arange(n, dtype=torch.float32)
    back = torch.full((n,), -1.0)
    tp = 2
    for t in range(tp):
        blk = registry.make_block(spec, tp, t)
        flat = torch.empty(blk.layout()[1])
        blk.load_from_whole(flat, ref)
        blk.store_into_whole(flat, back)
        rep = blk.tp_replicated_ranges()
        lay, _ = blk.layout()
        assert {o for o, _ in rep} == {lay["norm1_w"][0], lay["norm2_w"][0]}
        assert blk.num_params() < whole.num_params()
    lay, _ = whole.layout()
    for name, (o, sh) in lay.items():
        k = 1
        for d in sh:
            k *= d
        assert torch.equal(back[o:o + k], ref[o:o + k]), name


def test_checkpoint_across_tensor_parallel_widths(tmp_path):
    """Saved with tp 2: resumes with tp 2 and with tp 1 on two ZeRO ranks (blocks put back together
    from their slices); saved with tp 1 on two stages: resumes with tp 2."""
    from test_ckpt_health_cpu import _load_and_step, _train_and_save
    from test_dist_cpu import PIPE_1x2, PIPE_2x1

    ck = str(tmp_path / "ck")
    a = run_workers(2, _train_and_save, tiny_cfg(ONE_LANE, tensor_parallel_size=2), ck, 2)
    b = run_workers(2, _load_and_step, tiny_cfg(ONE_LANE, tensor_parallel_size=2), ck, 2)
    assert abs(a[0] - b[0]) < 1e-5, (a, b)
    d = run_workers(2, _load_and_step, tiny_cfg(PIPE_1x2), ck, 2)
    assert abs(a[0] - d[0]) < 1e-4, (a, d)
    ck1 = str(tmp_path / "ck1")
    e = run_workers(2, _train_and_save, tiny_cfg(PIPE_2x1), ck1, 2)
    f = run_workers(2, _load_and_step, tiny_cfg(ONE_LANE, tensor_parallel_size=2), ck1, 2)
    assert abs(e[0] - f[0]) < 1e-4, (e, f)


def test_parallel_dims_layout_and_training():
    """The four sizes give a valid config whose numbering inverts, and a 2 (shard) x 2 (tp) job from it
    trains like the oracle."""
    from zorse_b200.parallel.mesh import ParallelDims

    dims = ParallelDims(dp_replicate=2, dp_shard=2, tp=2, pp=3)
    assert dims.world_size == 24
    d = dims.training_config("tiny_llama", 4, 16, 2, 32, vocab_size=512)
    cfg = parse_pipeline_dict(d)
    assert cfg.world_size == 24 and len(cfg.stages) == 3
    assert cfg.stages[1].zero_config == ((4, 5), (6, 7))
    seen = set()
    for p in range(dims.world_size):
        c = dims.coordinates(p)
        assert p in dims.processes_of_lane(dims.lane(c["pp"], c["dp_replicate"], c["dp_shard"]))
        seen.add(tuple(c.values()))
    assert len(seen) == 24
    with pytest.raises(ValueError):
        ParallelDims(tp=0)
    small = ParallelDims(dp_shard=2, tp=2).training_config("tiny_llama", 4, 8, 2, 32, vocab_size=512,
                                                           autocast_dtype="float32", reduce_dtype="float32")
    res = run_workers(4, _worker, small, {"schedule": "layer_major"}, 2)
    _check_tp(res, small)


@pytest.mark.parametrize("model", ["toygpt", "deepspeedmistral_toy"])
def test_tp2_other_families(model):
    """LayerNorm + biases + GELU + learned positions (GPT), and grouped-query attention with a sliding
    window (Mistral): biases behind a reduce-scatter and the position table are lane-replicated."""
    cfg = tiny_cfg(ONE_LANE, tensor_parallel_size=2, model_name=model)
    res = run_workers(2, _worker, cfg, {"schedule": "layer_major"}, 2)
    _check_tp(res, cfg)


def _worker_ov(rank, world, cfg_dict, opts, overrides, steps):
    return _worker(rank, world, cfg_dict, dict(opts, model_overrides=overrides), steps)


def test_tp2_post_norm_block():
    """BERT-style layer (post-norm, LayerNorm, biases, embedding norm, learned positions), cut to two
    layers and a narrow width: residuals sit in front of the norms, so the residual gradient is added
    behind the reduce-scatter of the projection gradients."""
    from zorse_b200.models import registry
    from zorse_b200.utils.oracle import OracleTrainer

    ov = {"layers": 2, "hidden": 128, "heads": 4, "kv_heads": 4, "ffn": 256}
    pipe = [{"gpu_ranks": [0], "num_microbatches_per_rank": [4], "layer_partition": [0, 2], "zero_config": [[0]]}]
    cfg_dict = tiny_cfg(pipe, tensor_parallel_size=2, model_name="deepspeedbert_110m")
    res = run_workers(2, _worker_ov, cfg_dict, {"schedule": "layer_major"}, ov, 2)
    cfg = parse_pipeline_dict(cfg_dict)
    orc = OracleTrainer(cfg, model_overrides=ov)
    g = torch.Generator().manual_seed(7919)
    M, B, S = cfg.num_microbatches, cfg.microbatch_size, cfg.sequence_length
    batch = {"inputs": torch.randint(0, cfg.vocab_size, (M, B, S), generator=g),
             "targets": torch.randint(0, cfg.vocab_size, (M, B, S), generator=g)}
    want = [orc.step(batch) for _ in range(2)]
    spec = registry.get_spec(cfg.model_name, vocab=cfg.vocab_size, **ov)
    assert not spec.pre_norm
    for r in res:
        for a, b in zip(r["losses"], want):
            assert abs(a - b) < 2e-4, (r["losses"], want)
    for gid in (1, 2):
        whole = torch.zeros_like(orc.flats[gid])
        for r in res:
            registry.make_block(spec, 2, r["tp_index"]).store_into_whole(r["params"][gid], whole)
        assert (whole - orc.flats[gid].detach()).abs().max().item() < 5e-4


def test_scatter_gemm_bookkeeping_with_fake_kernels():
    """The slot offsets, flag indices, buffer parity and epochs `FusedTPComm` hands to its two kernels,
    checked by stand-ins that interpret device addresses in a fake address space: three processes, five
    operations with changing inputs, every result must equal the lane-wide sum of that operation."""
    from zorse_b200.parallel.tp_fused import FusedTPComm

    R, rows, H, K = 3, 256, 256, 64
    T = R * rows
    space = {}        # base address -> flat byte view

    def view_at(addr, nbytes):
        for base, buf in space.items():
            if base <= addr and addr + nbytes <= base + buf.numel():
                return buf[addr - base: addr - base + nbytes]
        raise AssertionError(f"address {addr} (+{nbytes}) outside every buffer")

    class Fake:
        def gemm_rs(self, a, b, *, b_mn, dst_ptrs, flag_ptrs, flag_index, epoch, counter, ldc, max_ctas=0):
            part = (a.float() @ (b.float() if b_mn else b.float().t())).to(torch.bfloat16)
            assert ldc == part.shape[1] and part.shape[0] % len(dst_ptrs) == 0
            n = part.shape[0] // len(dst_ptrs)
            for q, dst in enumerate(dst_ptrs):
                view_at(dst, n * ldc * 2).view(torch.bfloat16).copy_(part[q * n:(q + 1) * n].reshape(-1))
                view_at(flag_ptrs[q] + 4 * flag_index, 4).view(torch.int32).fill_(epoch)

        def rs_finish(self, slots, flags, R_, rows_, H_, epoch, out, resid=None, bias=None, wait_seconds=2.0):
            assert flags.numel() == R_ and int(flags.min()) >= epoch, (flags, epoch)   # a real kernel would wait
            acc = slots.view(R_, rows_, H_).float().sum(0)
            if resid is not None:
                acc = acc + resid.float()
            if bias is not None:
                acc = acc + bias.float()
            out.copy_(acc.to(out.dtype))
            return out

    def buffers_for(rank):
        def make(pg, size, device, stage_elems):
            return shared[rank]
        return make

    shared = []
    bases = []
    for r in range(R):
        stage = torch.zeros(2 * R * rows * H, dtype=torch.bfloat16)
        flags = torch.zeros(64, dtype=torch.int32)
        sb, fb = 1_000_000 * (r + 1), 1_000_000 * (r + 1) + 900_000
        space[sb] = stage.view(torch.uint8)
        space[fb] = flags.view(torch.uint8)
        bases.append((stage, flags, sb, fb))
    for r in range(R):
        shared.append((bases[r][0], bases[r][1], [b[2] for b in bases], [b[3] for b in bases]))
    comms = [FusedTPComm(None, R, r, device=torch.device("cpu"), rows=rows, hidden=H, kernels=Fake(),
                         buffers=buffers_for(r)) for r in range(R)]
    g = torch.Generator().manual_seed(0)
    for op in range(5):
        kmajor = op % 2 == 0
        xs = [torch.randn(T, K, generator=g).to(torch.bfloat16) for _ in range(R)]
        ws = [(torch.randn(H, K, generator=g) if kmajor else torch.randn(K, H, generator=g)).to(torch.bfloat16) for _ in range(R)]
        resid = [torch.randn(rows, H, generator=g).to(torch.bfloat16) for _ in range(R)]
        bias = torch.randn(H, generator=g).to(torch.bfloat16)
        parts = [(x.float() @ (w.float().t() if kmajor else w.float())).to(torch.bfloat16).float() for x, w in zip(xs, ws)]
        total = sum(parts)
        # every process sends, then every process finishes (the order real streams allow as well)
        ops_ = [comms[r].send(xs[r], ws[r], kmajor) for r in range(R)]
        outs = [comms[r].finish(ops_[r], resid[r] if op % 3 else None, bias if op % 2 else None) for r in range(R)]
        for r in range(R):
            want = total[r * rows:(r + 1) * rows]
            if op % 3:
                want = want + resid[r].float()
            if op % 2:
                want = want + bias.float()
            assert (outs[r].float() - want).abs().max().item() < 0.51, (op, r)
    assert all(c.n_ops == 5 for c in comms)


def test_fused_lane_gather_and_scatter_protocol_with_threads():
    """The whole fused-lane protocol (scatter GEMM -> sum + norm + push -> gathered buffers, buffer parity,
    flag indices, epochs) with stand-in kernels over a fake address space, one thread per process so that a
    fast process really can run ahead: every gathered tensor must hold the rows of the operation it belongs
    to.  The stand-ins wait on flags by polling, as the kernels do."""
    import threading
    import time

    from zorse_b200.ops.api import get_ops
    from zorse_b200.parallel.tp_fused import FusedTPComm

    R, rows, H, K = 3, 256, 256, 32
    T = R * rows
    space = {}

    def view_at(addr, nbytes):
        for base, buf in space.items():
            if base <= addr and addr + nbytes <= base + buf.numel():
                return buf[addr - base: addr - base + nbytes]
        raise AssertionError(f"address {addr} (+{nbytes}) outside every buffer")

    def poll(flags, want):
        t0 = time.time()
        while int(flags.min()) < want:
            assert time.time() - t0 < 20, "flag never arrived"
            time.sleep(0.0005)

    def rms(x, w, eps=1e-5):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(torch.bfloat16)

    class Fake:
        def gemm_rs(self, a, b, *, b_mn, dst_ptrs, flag_ptrs, flag_index, epoch, counter, ldc, max_ctas=0):
            part = (a.float() @ (b.float() if b_mn else b.float().t())).to(torch.bfloat16)
            n = part.shape[0] // len(dst_ptrs)
            for q, dst in enumerate(dst_ptrs):
                view_at(dst, n * ldc * 2).view(torch.bfloat16).copy_(part[q * n:(q + 1) * n].reshape(-1))
            for q in range(len(dst_ptrs)):
                view_at(flag_ptrs[q] + 4 * flag_index, 4).view(torch.int32).fill_(epoch)

        def rs_finish(self, *a, **k):
            raise AssertionError("not used in this test")

        def wait_flags(self, flags, R_, which, epoch, wait_seconds=2.0):
            poll(flags[which * R_:(which + 1) * R_], epoch)

        def _push(self, y, dst_ptrs, flag_ptrs, flag_index, epoch):
            for dst in dst_ptrs:
                view_at(dst, y.numel() * 2).view(torch.bfloat16).copy_(y.reshape(-1))
            for q in range(len(dst_ptrs)):
                view_at(flag_ptrs[q] + 4 * flag_index, 4).view(torch.int32).fill_(epoch)

        def tp_push(self, src, dst_ptrs, flag_ptrs, flag_index, epoch, counter):
            self._push(src, dst_ptrs, flag_ptrs, flag_index, epoch)

        def tp_norm_push(self, *, w, b, eps, layernorm, y_local, dst_ptrs, flag_ptrs, flag_index, epoch, stats, counter,
                         x=None, slots=None, in_flags=None, in_epoch=0, resid=None, bias=None, h_out=None, wait_seconds=2.0):
            assert not layernorm
            if slots is not None:
                poll(in_flags, in_epoch)
                acc = slots.view(-1, *y_local.shape).float().sum(0)
                if resid is not None:
                    acc = acc + resid.float()
                h_out.copy_(acc.to(torch.bfloat16))
                x = h_out
            y_local.copy_(rms(x, w, eps))
            self._push(y_local, dst_ptrs, flag_ptrs, flag_index, epoch)

    bases = []
    for r in range(R):
        stage = torch.zeros(4 * R * rows * H, dtype=torch.bfloat16)
        flags = torch.zeros(64, dtype=torch.int32)
        sb, fb = 100_000_000 * (r + 1), 100_000_000 * (r + 1) + 90_000_000
        space[sb], space[fb] = stage.view(torch.uint8), flags.view(torch.uint8)
        bases.append((stage, flags, sb, fb))
    shared = [(bases[r][0], bases[r][1], [b[2] for b in bases], [b[3] for b in bases]) for r in range(R)]
    comms = [FusedTPComm(None, R, r, device=torch.device("cpu"), rows=rows, hidden=H, kernels=Fake(),
                         buffers=(lambda rr: (lambda pg, size, device, n: shared[rr]))(r)) for r in range(R)]
    g = torch.Generator().manual_seed(3)
    rounds = 4
    w1 = (1 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    data = [[{"x": torch.randn(rows, H, generator=g).to(torch.bfloat16), "a": torch.randn(T, K, generator=g).to(torch.bfloat16),
              "w": torch.randn(H, K, generator=g).to(torch.bfloat16), "res": torch.randn(rows, H, generator=g).to(torch.bfloat16),
              "y": torch.randn(rows, H, generator=g).to(torch.bfloat16)} for _ in range(R)] for _ in range(rounds)]
    got = [[None] * R for _ in range(rounds)]
    errors = []
    ops = get_ops("ref")

    def program(r):
        try:
            c = comms[r]
            for k in range(rounds):
                d = data[k][r]
                if r == k % R:
                    time.sleep(0.02)                     # somebody is always late
                n, st, n_all = c.norm_gather(ops, d["x"], w1, None, 1e-5, "rms")
                n_all = n_all.clone()
                h, n2, st2, n2_all = c.linear_rs_norm_gather(ops, d["a"], d["w"], True, d["res"], None, w1, None, 1e-5, "rms")
                n2_all = n2_all.clone()
                y_all = c.gather_rows(d["y"]).clone()
                got[k][r] = (n_all, h.clone(), n2_all, y_all)
        except Exception as e:      # noqa: BLE001 - reported through the list
            errors.append((r, repr(e)))

    ths = [threading.Thread(target=program, args=(r,)) for r in range(R)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(120)
    assert not errors, errors
    for k in range(rounds):
        want_n = torch.cat([rms(data[k][q]["x"], w1) for q in range(R)])
        parts = [(data[k][q]["a"].float() @ data[k][q]["w"].float().t()).to(torch.bfloat16).float() for q in range(R)]
        total = sum(parts)
        hs = [(total[q * rows:(q + 1) * rows] + data[k][q]["res"].float()).to(torch.bfloat16) for q in range(R)]
        want_n2 = torch.cat([rms(h, w1) for h in hs])
        want_y = torch.cat([data[k][q]["y"] for q in range(R)])
        for r in range(R):
            n_all, h, n2_all, y_all = got[k][r]
            assert torch.equal(n_all, want_n), (k, r, "norm gather")
            assert torch.equal(h, hs[r]), (k, r, "reduce-scatter sum")
            assert torch.equal(n2_all, want_n2), (k, r, "sum + norm gather")
            assert torch.equal(y_all, want_y), (k, r, "plain gather")


def test_take_and_put_slice_are_inverse_for_random_cuts():
    """Property: for random segment layouts, widths and cut dimensions the slices of all processes tile the
    tensor exactly once and put_slice restores it."""
    from hypothesis import given, settings, strategies as st

    from zorse_b200.models.tp_layers import put_slice, take_slice

    @settings(max_examples=60, deadline=None)
    @given(tp=st.sampled_from([1, 2, 3, 4]), segs=st.lists(st.integers(1, 5), min_size=1, max_size=3),
           other=st.integers(1, 4), dim=st.sampled_from([0, 1]))
    def check(tp, segs, other, dim):
        segments = tuple(s * tp for s in segs)
        shape = (sum(segments), other) if dim == 0 else (other, sum(segments))
        full = torch.arange(shape[0] * shape[1], dtype=torch.float32).view(shape)
        back = torch.full(shape, -1.0)
        seen = []
        for t in range(tp):
            piece = take_slice(full, dim, segments, tp, t)
            assert piece.shape[dim] == sum(segments) // tp and piece.shape[1 - dim] == other
            seen.append(piece.reshape(-1))
            put_slice(back, piece, dim, segments, tp, t)
        assert torch.equal(back, full)
        assert sorted(torch.cat(seen).tolist()) == full.reshape(-1).tolist()

    check()


def _worker_gpu_ops_dry_run(rank, world, cfg_dict):
    """One step of a tensor-parallel lane through the GPU op layer on a stand-in library (CPU tensors)."""
    from test_sm100_wrappers_cpu import FakeLib, c_prototypes
    from zorse_b200.ops import sm100 as k
    from zorse_b200.trainer import Trainer, TrainerOptions

    fake = FakeLib()
    k._lib = fake
    k._bf16 = lambda t, name: None
    k.status_word = lambda device=None: torch.zeros(1, dtype=torch.int32)
    k._stream = lambda: None
    k.check_status = lambda device=None: None
    tr = Trainer(parse_pipeline_dict(cfg_dict), TrainerOptions(backend="gloo", schedule="1f1b", ops="sm100",
                                                               activation_recompute=False))
    tr.train_step_from_host(tr.synthetic_batch())
    protos = c_prototypes()
    bad = [(n, a, protos.get(n)) for n, a in fake.calls if protos.get(n) != a]
    return {"calls": len(fake.calls), "bad": bad, "names": sorted({n for n, _ in fake.calls})}


@pytest.mark.parametrize("layout", ["tp2", "two_stages", "zero2way"])
def test_tp_lane_through_the_gpu_op_layer_dry_run(layout):
    """... and the same for two pipeline stages and for a two-way ZeRO stage (bf16 tensors over gloo)."""
    from test_dist_cpu import PIPE_1x2, PIPE_2x1

    pipe, tp = {"tp2": (ONE_LANE, 2), "two_stages": (PIPE_2x1, 1), "zero2way": (PIPE_1x2, 1)}[layout]
    cfg = tiny_cfg(pipe, tensor_parallel_size=tp, autocast_dtype="bfloat16", reduce_dtype="bfloat16", sequence_length=128)
    res = run_workers(2, _worker_gpu_ops_dry_run, cfg)
    for r in res:
        assert r["calls"] > 100 and not r["bad"], r["bad"]
        names = set(r["names"])
        assert names & {"zb_flash_fwd", "zb_flash_fwd4"} and names & {"zb_norm_bwd", "zb_norm_bwd2"}   # whichever versions are default
