"""Single-process oracle trainer: the same model as one autograd graph in fp32 on the CPU.

It builds every layer of the model from the same seeds as the engine, runs the layers'
`forward` through the PyTorch ops under autograd, takes the mean cross-entropy over the
whole global batch and steps `torch.optim.Adam`.  Distributed runs (any stage split, DP
width, schedule) are compared against it: loss, and parameters after a few steps.
"""
from __future__ import annotations

import torch

from ..config.training_config import PipelineConfig
from ..models import registry
from ..ops.api import get_ops


class OracleTrainer:
    def __init__(self, cfg: PipelineConfig, seed: int = 0, lr: float = 1e-3, dtype=torch.float32, model_overrides=None):
        self.cfg = cfg
        self.ops = get_ops("ref")
        self.spec = registry.get_spec(cfg.model_name, vocab=cfg.vocab_size, **(model_overrides or {}))
        self.layers = registry.build_stage_layers(self.spec, 0, self.spec.layers, cfg.sequence_length)
        self.flats = []
        for i, ly in enumerate(self.layers):
            gid = registry.global_layer_index(self.spec, 0, i, self.layers)
            _, n = ly.layout()
            flat = torch.empty(n, dtype=torch.float32)
            ly.init_flat(flat, seed * 1000003 + gid)
            flat = flat.to(dtype).requires_grad_(True)
            self.flats.append(flat)
        self.opt = torch.optim.Adam(self.flats, lr=lr, betas=(0.9, 0.999), eps=1e-8)

    def loss(self, batch) -> torch.Tensor:
        cfg = self.cfg
        M = cfg.num_microbatches
        total = 0.0
        for g in range(M):
            x = batch["inputs"][g]
            B = x.shape[0]
            S = cfg.sequence_length
            if self.spec.family == "vit":
                S = self.layers[0].tokens_per_image()
            for ly, flat in zip(self.layers, self.flats):
                ly.bind(flat, None)
                ctx = {"B": B, "S": S, "loss_scale": 1.0}
                if ly.kind == "head":
                    ctx["targets"] = batch["targets"][g]
                x = ly.forward(x, ctx, self.ops, None)
            total = total + x.float().mean() / M
        return total

    def step(self, batch) -> float:
        self.opt.zero_grad(set_to_none=True)
        loss = self.loss(batch)
        loss.backward()
        self.opt.step()
        return float(loss.detach())

    def grads(self, batch):
        for f in self.flats:
            f.grad = None
        loss = self.loss(batch)
        loss.backward()
        return float(loss.detach()), [f.grad.clone() for f in self.flats]
