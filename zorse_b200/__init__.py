"""zorse-b200: hybrid pipeline-parallel + ZeRO (+ tensor-parallel) LLM training for B200 nodes.

    from zorse_b200 import Trainer, TrainerOptions, parse_pipeline_config

    trainer = Trainer(parse_pipeline_config("training_config.json"), TrainerOptions(schedule="1f1b"))
    batch = trainer.synthetic_batch()
    loss = trainer.train_step_from_host(batch)

The names below are loaded on first use, so that `import zorse_b200` stays cheap for the tools that only
need the configuration reader or the planner.
"""
__version__ = "0.1.0"

_LAZY = {
    "Trainer": ("zorse_b200.trainer", "Trainer"),
    "TrainerOptions": ("zorse_b200.trainer", "TrainerOptions"),
    "parse_pipeline_config": ("zorse_b200.config.training_config", "parse_pipeline_config"),
    "parse_pipeline_dict": ("zorse_b200.config.training_config", "parse_pipeline_dict"),
    "PipelineConfig": ("zorse_b200.config.training_config", "PipelineConfig"),
    "ParallelDims": ("zorse_b200.parallel.mesh", "ParallelDims"),
    "save_checkpoint": ("zorse_b200.ckpt.writer", "save_checkpoint"),
    "load_checkpoint": ("zorse_b200.ckpt.reader", "load_checkpoint"),
}

__all__ = ["__version__", *_LAZY]


def __getattr__(name):
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        return getattr(importlib.import_module(mod), attr)
    raise AttributeError(f"module 'zorse_b200' has no attribute {name!r}")
