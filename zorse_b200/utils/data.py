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


def split_into(inputs: torch.Tensor, labels: torch.Tensor, microbatches: int):
    """A batch cut into `microbatches` pieces whose sizes differ by at most one sample, larger pieces first
    (reference utils/data_loader.py:54-67, which takes a COUNT where `split_microbatches` above takes a size)."""
    n = len(inputs)
    base, rem = divmod(n, microbatches)
    if base == 0:
        raise ValueError(f"{n} samples cannot fill {microbatches} microbatches")
    sizes = [base + (1 if i < rem else 0) for i in range(microbatches)]
    return inputs.split(sizes), labels.split(sizes)


class RandomTokenDataset(torch.utils.data.Dataset):
    """`size` random token sequences, generated once from `seed`.  `targets`: "next" = the input shifted by one with
    a fresh random last token (language modelling), "random" = independent random tokens, "regression" = one float in
    [0, 1) per position.  Covers the reference's three toy datasets for sequences
    (utils/data_loader.py:70-90, 116-144) and its TensorDataset of random batches (:31-38)."""

    def __init__(self, vocab_size: int, seq_length: int, size: int = 1000, targets: str = "next", seed: int = 0):
        if targets not in ("next", "random", "regression"):
            raise ValueError(f"targets must be next, random or regression, not {targets!r}")
        g = torch.Generator().manual_seed(seed)
        self.inputs = torch.randint(0, vocab_size, (size, seq_length), generator=g)
        if targets == "next":
            self.labels = torch.cat([self.inputs[:, 1:], torch.randint(0, vocab_size, (size, 1), generator=g)], dim=1)
        elif targets == "random":
            self.labels = torch.randint(0, vocab_size, (size, seq_length), generator=g)
        else:
            self.labels = torch.rand(size, seq_length, generator=g)

    def __len__(self) -> int:
        return len(self.inputs)

    def __getitem__(self, i):
        return self.inputs[i], self.labels[i]


class RandomImageDataset(torch.utils.data.Dataset):
    """`size` random images with a class id (`classes` > 0) or a regression target in [0, 1) (`classes` = 0)
    (reference utils/data_loader.py:41-51, 93-113)."""

    def __init__(self, image_size: int, channels: int = 3, size: int = 1000, classes: int = 2, seed: int = 0,
                 dtype: torch.dtype = torch.float32):
        g = torch.Generator().manual_seed(seed)
        self.images = torch.randn(size, channels, image_size, image_size, generator=g).to(dtype)
        self.labels = (torch.randint(0, classes, (size,), generator=g) if classes > 0
                       else torch.rand(size, generator=g).to(dtype))

    def __len__(self) -> int:
        return len(self.images)

    def __getitem__(self, i):
        return self.images[i], self.labels[i]


def get_dataset(model_name: str, *, batch_size: int, batches: int, seq_length: int = 512, vocab_size: int = 32000,
                image_size: int = 224, seed: int = 0) -> torch.utils.data.DataLoader:
    """A loader of `batches` random batches for the model: images for vision models, token ids otherwise
    (reference utils/data_loader.py:24-51 sizes it as warm-up + timed iterations)."""
    from ..models import registry

    if registry.get_spec(model_name).family == "vit":
        ds = RandomImageDataset(image_size, size=batches * batch_size, seed=seed)
    else:
        ds = RandomTokenDataset(vocab_size, seq_length, size=batches * batch_size, targets="random", seed=seed)
    return torch.utils.data.DataLoader(ds, batch_size=batch_size)


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
