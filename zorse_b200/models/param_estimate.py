"""Closed-form parameter counts per model (reference models/param_estimate.py).

    python -m zorse_b200.models.param_estimate --model_name llama2_7b [--vocab_size 32000] [--seq_length 4096]
"""
from __future__ import annotations

import argparse

from . import registry


def estimate(name: str, vocab_size=None, seq_length: int = 0) -> dict:
    s = registry.get_spec(name, vocab=vocab_size)
    H, F, D = s.hidden, s.ffn, s.head_dim
    qkv = (s.heads + 2 * s.n_kv) * D * H
    attn = qkv + s.heads * D * H
    mlp = (3 if s.act == "swiglu" else 2) * H * F
    norms = 2 * H * (2 if s.norm == "ln" else 1)
    bias = ((s.heads + 2 * s.n_kv) * D + H + (2 * F if s.act == "swiglu" else F) + H) if s.bias else 0
    per_layer = attn + mlp + norms + bias
    assert per_layer == registry.params_per_block(s), (per_layer, registry.params_per_block(s))
    total = registry.total_params(s, seq_length)
    return {"model": name, "layers": s.layers, "parameters_per_layer": per_layer, "attention": attn, "mlp": mlp,
            "embedding_and_head": total - s.layers * per_layer, "total_parameters": total}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_name", required=True)
    ap.add_argument("--vocab_size", type=int, default=None)
    ap.add_argument("--seq_length", type=int, default=0)
    a = ap.parse_args(argv)
    for k, v in estimate(a.model_name, a.vocab_size, a.seq_length).items():
        print(f"{k:24s} {v}")


if __name__ == "__main__":
    main()
