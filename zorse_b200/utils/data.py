"""Synthetic data helpers (reference utils/data_loader.py:7-144, utils/loss_funcs.py)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def generate_model_data(model_name: str, batch_size: int, seq_length: int, vocab_size: int = 32000, image_size: int = 384,
                        device="cpu", seed: int = 0):
    """(inputs, targets) for one batch: token ids for language models, images + class ids for ViT."""
    from ..models import registry

    g = torch.Generator().manual_seed(seed)
    spec = registry.get_spec(model_name)
    if spec.family == "vit":
        x = torch.randn(batch_size, 3, image_size, image_size, generator=g)
        y = torch.randint(0, spec.classes, (batch_size,), generator=g)
    else:
        x = torch.randint(0, vocab_size, (batch_size, seq_length), generator=g)
        y = torch.randint(0, vocab_size, (batch_size, seq_length), generator=g)
    return x.to(device), y.to(device)


def split_microbatches(t: torch.Tensor, microbatch_size: int) -> list[torch.Tensor]:
    return list(t.split(microbatch_size, dim=0))


def shift_labels(tokens: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Next-token targets for real text: target[t] = token[t+1], last position ignored."""
    y = torch.full_like(tokens, ignore_index)
    y[..., :-1] = tokens[..., 1:]
    return y


class LMLoss(torch.nn.Module):
    def forward(self, logits, targets):
        return F.cross_entropy(logits.flatten(0, -2).float(), targets.flatten())


class RegressionLoss(torch.nn.Module):
    def forward(self, out, targets):
        return F.mse_loss(out.float(), targets.float())
