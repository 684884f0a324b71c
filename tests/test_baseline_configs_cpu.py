"""Scaled-down versions of the named benchmark configurations 2, 3, 4 and 5 on CPU ranks (gloo):
same model families, parallel plans and engine options, tiny dimensions; each must reproduce
the single-process oracle (loss and parameters after two steps)."""
import torch

from dist_utils import run_workers
from zorse_b200.config.training_config import parse_pipeline_dict


def _worker(rank, world, cfg_dict, opts, overrides, steps):
    from zorse_b200.trainer import Trainer, TrainerOptions

    cfg = parse_pipeline_dict(cfg_dict)
    tr = Trainer(cfg, TrainerOptions(backend="gloo", model_overrides=overrides, **opts))
    batch = tr.synthetic_batch()
    losses = [tr.global_loss(tr.train_step_from_host(batch)) for _ in range(steps)]
    params = {u.gid: u.full_master()[: u.layer.layout()[1]].clone() for st in tr.stages for u in st.engine.units}
    cnt = [(c.h2d_bytes, c.d2h_bytes) for c in tr.counters()]
    return {"losses": losses, "params": params, "offload_bytes": cnt}


def _oracle(cfg_dict, overrides, steps):
    from zorse_b200.utils.oracle import OracleTrainer

    cfg = parse_pipeline_dict(cfg_dict)
    orc = OracleTrainer(cfg, model_overrides=overrides)
    g = torch.Generator().manual_seed(7919)
    M, B, S = cfg.num_microbatches, cfg.microbatch_size, cfg.sequence_length
    batch = {"inputs": torch.randint(0, cfg.vocab_size, (M, B, S), generator=g),
             "targets": torch.randint(0, cfg.vocab_size, (M, B, S), generator=g)}
    return [orc.step(batch) for _ in range(steps)], [f.detach() for f in orc.flats]


def _check(results, cfg_dict, overrides, steps=2):
    want_losses, want_params = _oracle(cfg_dict, overrides, steps)
    for res in results:
        for a, b in zip(res["losses"], want_losses):
            assert abs(a - b) < 3e-4, (res["losses"], want_losses)
        for gid, p in res["params"].items():
            err = (p - want_params[gid]).abs().max().item()
            assert err < 6e-4, f"unit {gid}: max param error {err}"


def _cfg(model, pipe, gbs, mbs, seq, vocab, **kw):
    d = {"model_name": model, "global_batch_size": gbs, "microbatch_size": mbs, "sequence_length": seq,
         "vocab_size": vocab, "autocast_dtype": "float32", "reduce_dtype": "float32", "pipeline_config": pipe}
    d.update(kw)
    return d


def test_config2_like_gqa_two_stages_zero2_optimizer_in_backward():
    """Llama-3.2-1B plan (2 stages x 2-way ZeRO-2, GQA 4:1, optimizer in backward), tiny dimensions."""
    ov = {"layers": 4, "hidden": 128, "heads": 8, "kv_heads": 2, "ffn": 256}
    pipe = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [2, 2], "layer_partition": [0, 2],
             "zero_config": [[0, 1]], "zero_level": 2},
            {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [2, 2], "layer_partition": [2, 4],
             "zero_config": [[2, 3]], "zero_level": 2}]
    cfg = _cfg("llama3.2_1b", pipe, 8, 2, 32, 512)
    res = run_workers(4, _worker, cfg, {"schedule": "zero2", "optimizer_in_backward": True}, ov, 2)
    _check(res, cfg, ov)


def test_config3_like_four_stages_two_way_zero3_as_the_benchmark_runs_it():
    """The headline plan (4 stages x 2-way ZeRO-3 on 8 ranks) with the options `bench.py` picks for it: 1F1B without
    recomputation, weight gradients of the head and the last block of the last stage held back to the end of its
    backward; and once more under the schedule the configuration names (ZeRO-2 pipeline schedule, recomputing)."""
    ov = {"layers": 8, "hidden": 64, "heads": 4, "kv_heads": 4, "ffn": 128}
    pipe = [{"gpu_ranks": [2 * i, 2 * i + 1], "num_microbatches_per_rank": [4, 4], "layer_partition": [2 * i, 2 * i + 2],
             "zero_config": [[2 * i, 2 * i + 1]]} for i in range(4)]
    cfg = _cfg("llama2_7b", pipe, 8, 1, 32, 512)
    res = run_workers(8, _worker, cfg, {"schedule": "1f1b", "defer_tail_wgrad": 2, "activation_recompute": False}, ov, 2)
    _check(res, cfg, ov)
    res = run_workers(8, _worker, cfg, {"schedule": "zero2"}, ov, 2)
    _check(res, cfg, ov)


def test_config4_like_mistral_sliding_window_uneven_split():
    """Mistral plan (2 stages x 2-way ZeRO-3, uneven 1/3 layer split, sequence longer than the window)."""
    pipe = [{"gpu_ranks": [0, 1], "num_microbatches_per_rank": [2, 2], "layer_partition": [0, 1], "zero_config": [[0, 1]]},
            {"gpu_ranks": [2, 3], "num_microbatches_per_rank": [2, 2], "layer_partition": [1, 4], "zero_config": [[2, 3]]}]
    ov = {"hidden": 128, "heads": 8, "kv_heads": 2, "ffn": 256, "window": 16}
    cfg = _cfg("deepspeedmistral_toy", pipe, 4, 1, 48, 512)
    res = run_workers(4, _worker, cfg, {"schedule": "layer_major"}, ov, 2)
    _check(res, cfg, ov)


def test_config5_like_opt_four_stages_parameter_offload():
    """OPT plan (one rank per stage, parameters offloaded to the host, optimizer in backward)."""
    ov = {"layers": 4, "hidden": 64, "heads": 4, "ffn": 256, "max_positions": 64}
    pipe = [{"gpu_ranks": [r], "num_microbatches_per_rank": [4], "layer_partition": [r, r + 1], "zero_config": [[r]]}
            for r in range(4)]
    cfg = _cfg("opt_125m", pipe, 8, 2, 32, 512)
    res = run_workers(4, _worker, cfg, {"schedule": "zero2", "optimizer_in_backward": True,
                                        "offload_model_params": True}, ov, 2)
    _check(res, cfg, ov)
    assert all(h > 0 and d > 0 for r in res for (h, d) in r["offload_bytes"])
