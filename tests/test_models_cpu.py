"""Every model family: the layers' explicit backward passes (through the PyTorch ops backend)
must reproduce autograd of the same forward, for the whole model, after an optimizer step."""
import pytest

from zorse_b200.config.training_config import parse_pipeline_dict
from zorse_b200.trainer import Trainer, TrainerOptions
from zorse_b200.utils.oracle import OracleTrainer

FAMILIES = [
    ("tiny_llama", {"layers": 2, "hidden": 64, "heads": 4, "ffn": 96}, 16),
    ("deepspeedllamav2_tiny", {"layers": 2, "hidden": 64, "heads": 4, "ffn": 96}, 16),
    ("deepspeedmistral_toy", {"layers": 2, "hidden": 64, "heads": 4, "kv_heads": 2, "ffn": 96, "window": 5}, 16),
    ("toygpt_small", {"layers": 2, "hidden": 64, "heads": 4, "ffn": 128}, 16),
    ("opt_125m", {"layers": 2, "hidden": 64, "heads": 4, "ffn": 128, "max_positions": 32}, 16),
    ("deepspeedbert_base", {"layers": 2, "hidden": 64, "heads": 4, "ffn": 128, "max_positions": 32}, 16),
    ("deepspeedvit_default", {"layers": 2, "hidden": 64, "heads": 4, "ffn": 128, "image": 32, "patch": 8}, 17),
]


@pytest.mark.parametrize("model,ov,seq", FAMILIES)
@pytest.mark.parametrize("schedule", ["layer_major", "1f1b"])
def test_family_matches_autograd(model, ov, seq, schedule):
    nl = ov["layers"]
    cfg = parse_pipeline_dict({
        "model_name": model, "global_batch_size": 4, "microbatch_size": 2, "sequence_length": seq, "vocab_size": 128,
        "autocast_dtype": "float32", "reduce_dtype": "float32",
        "pipeline_config": [{"gpu_ranks": [0], "num_microbatches_per_rank": [2], "layer_partition": [0, nl],
                             "zero_config": [[0]]}]})
    tr = Trainer(cfg, TrainerOptions(schedule=schedule, model_overrides=ov, ops="ref"))
    orc = OracleTrainer(cfg, model_overrides=ov)
    batch = tr.synthetic_batch()
    for _ in range(2):
        loss = tr.train_step_from_host(batch)
        want = orc.step(batch)
    assert abs(loss - want) < 1e-4 * max(1.0, abs(want)), (loss, want)
    for u, f in zip(tr.stages[0].engine.units, orc.flats):
        err = (u.full_master()[: f.numel()] - f.detach()).abs().max().item()
        assert err < 5e-4, f"{model} unit {u.gid} ({u.layer.kind}): {err}"


def test_registry_lists_every_reference_family():
    from zorse_b200.models import registry

    names = registry.list_models()
    for prefix in ("deepspeedllama_", "deepspeedllamav2_", "deepspeedmistral_", "deepspeedgpt_", "toygpt", "opt_",
                   "deepspeedbert_", "deepspeedvit_"):
        assert any(n.startswith(prefix) for n in names), prefix


def test_model_stats_file_matches_registry():
    """data/model_stats.json is generated from the registry (python -m zorse_b200.models.registry)."""
    import json
    from pathlib import Path

    from zorse_b200.models import registry

    path = Path(__file__).resolve().parents[1] / "data" / "model_stats.json"
    table = json.loads(path.read_text())
    assert sorted(table) == registry.list_models()
    for name in ("llama2_7b", "deepspeedgpt_1.3b", "opt_13b", "deepspeedbert_large", "deepspeedvit_g"):
        assert table[name] == registry.get_model_stats(name)
    # figure quoted by the reference's own table for a Llama-7B block
    assert table["deepspeedllama_7b"]["parameters_per_layer"] == 202383360


def test_example_files_parse():
    import json
    from pathlib import Path

    from zorse_b200.config.training_config import parse_pipeline_config
    from zorse_b200.profiler.cluster import read_machine_file

    ex = Path(__file__).resolve().parents[1] / "example"
    cfg = parse_pipeline_config(ex / "training_config.json")
    assert cfg.model_name == "llama2_7b" and len(cfg.stages) == 4 and cfg.num_microbatches == 64
    info = json.loads((ex / "cluster_info.json").read_text())
    assert info["total_gpus"] == 8
    hosts = read_machine_file(str(ex / "hostfile"))
    assert len(hosts) == 1 and hosts[0].local
