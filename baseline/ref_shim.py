"""Compatibility shim that lets the unmodified reference tree import and run against the
installed transformers / torch.  Nothing in the reference tree is edited: this module only
adds names that newer library versions removed, before the reference imports them.

What the reference imports and the installed libraries no longer provide:

* `transformers.models.llama.modeling_llama.LlamaFlashAttention2` / `LlamaSdpaAttention`
  (reference `models/llama_simple.py:7-13`, chosen per layer at `models/llama_simple.py:396-416`).
  The stand-ins below restate what those classes did in the transformers release the reference
  was written for: separate q/k/v/o projections, rotary embedding from `position_ids`, then
  flash-attn 2 (`flash_attn_func`, causal) or `torch.nn.functional.scaled_dot_product_attention`
  (causal).  Both return the reference's `(attn_output, attn_weights, past_key_value)` triple.
* `transformers.pytorch_utils.find_pruneable_heads_and_indices` / `prune_conv1d_layer`
  (reference `models/gpt_simple.py:6-10`; only head pruning uses them, which no training path calls).

Run-time table rows (reference `utils/train_utils.py:245-273`, `utils/runtime_estimator.py:22-38`)
for the B200 and for bf16 are added by `patch_tables()` after the reference modules are imported.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn


def _rope_theta(config) -> float:
    theta = getattr(config, "rope_theta", None)
    if theta is None:
        params = getattr(config, "rope_parameters", None) or getattr(config, "rope_scaling", None) or {}
        theta = params.get("rope_theta", 10000.0) if isinstance(params, dict) else 10000.0
    return float(theta)


class _RotaryEmbedding(nn.Module):
    """cos/sin of shape [batch, seq, head_dim] from position ids, computed in fp32 and cast to the
    activation dtype (the arithmetic of the reference's own `LlamaRotaryEmbedding`,
    `models/llama_simple.py:61-137`)."""

    def __init__(self, dim: int, base: float):
        super().__init__()
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.int64).float() / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)

    @torch.no_grad()
    def forward(self, x, position_ids):
        inv = self.inv_freq[None, :, None].float().expand(position_ids.shape[0], -1, 1).to(x.device)
        pos = position_ids[:, None, :].float()
        with torch.autocast(device_type=x.device.type, enabled=False):
            freqs = (inv @ pos).transpose(1, 2)
            emb = torch.cat((freqs, freqs), dim=-1)
            cos, sin = emb.cos(), emb.sin()
        return cos.to(dtype=x.dtype), sin.to(dtype=x.dtype)


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


class _LlamaAttentionBase(nn.Module):
    def __init__(self, config, layer_idx=None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = self.hidden_size // self.num_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.is_causal = True
        bias = bool(getattr(config, "attention_bias", False))
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=bias)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=bias)
        self.o_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=bias)
        self.rotary_emb = _RotaryEmbedding(self.head_dim, _rope_theta(config))

    def _qkv(self, hidden_states, position_ids):
        b, s, _ = hidden_states.shape
        q = self.q_proj(hidden_states).view(b, s, self.num_heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(hidden_states).view(b, s, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(hidden_states).view(b, s, self.num_key_value_heads, self.head_dim).transpose(1, 2)
        cos, sin = self.rotary_emb(v, position_ids)
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
        q = (q * cos) + (_rotate_half(q) * sin)
        k = (k * cos) + (_rotate_half(k) * sin)
        return q, k, v


class LlamaFlashAttention2(_LlamaAttentionBase):
    """flash-attn 2 path (library kernel), as the reference selects for half-precision dtypes."""

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False, cache_position=None, **kwargs):
        from flash_attn import flash_attn_func

        b, s, _ = hidden_states.shape
        q, k, v = self._qkv(hidden_states, position_ids)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)     # flash-attn wants [b, s, h, d]
        if q.dtype == torch.float32:
            tgt = torch.get_autocast_gpu_dtype() if torch.is_autocast_enabled() else self.q_proj.weight.dtype
            if tgt == torch.float32:
                tgt = torch.bfloat16
            q, k, v = q.to(tgt), k.to(tgt), v.to(tgt)
        out = flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=True)
        out = out.reshape(b, s, self.hidden_size).contiguous()
        return self.o_proj(out), None, past_key_value


class LlamaSdpaAttention(_LlamaAttentionBase):
    """`scaled_dot_product_attention` path (torch picks its own fused backend)."""

    def forward(self, hidden_states, attention_mask=None, position_ids=None, past_key_value=None,
                output_attentions=False, use_cache=False, cache_position=None, **kwargs):
        b, s, _ = hidden_states.shape
        q, k, v = self._qkv(hidden_states, position_ids)
        if self.num_key_value_groups > 1:
            k = k.repeat_interleave(self.num_key_value_groups, dim=1)
            v = v.repeat_interleave(self.num_key_value_groups, dim=1)
        out = torch.nn.functional.scaled_dot_product_attention(
            q.contiguous(), k.contiguous(), v.contiguous(), attn_mask=None, dropout_p=0.0, is_causal=True)
        out = out.transpose(1, 2).contiguous().view(b, s, self.hidden_size)
        return self.o_proj(out), None, past_key_value


def _find_pruneable_heads_and_indices(heads, n_heads, head_size, already_pruned_heads):
    mask = torch.ones(n_heads, head_size)
    heads = set(heads) - already_pruned_heads
    for head in heads:
        head = head - sum(1 if h < head else 0 for h in already_pruned_heads)
        mask[head] = 0
    mask = mask.view(-1).contiguous().eq(1)
    index = torch.arange(len(mask))[mask].long()
    return heads, index


def _prune_conv1d_layer(layer, index, dim=1):
    from transformers.pytorch_utils import Conv1D

    index = index.to(layer.weight.device)
    w = layer.weight.index_select(dim, index).detach().clone()
    b = layer.bias.detach().clone() if dim == 0 else layer.bias[index].detach().clone()
    new_size = list(layer.weight.size())
    new_size[dim] = len(index)
    new_layer = Conv1D(new_size[1], new_size[0]).to(layer.weight.device)
    with torch.no_grad():
        new_layer.weight.copy_(w.contiguous())
        new_layer.bias.copy_(b.contiguous())
    return new_layer


def install() -> list:
    """Adds the removed names to the installed transformers modules.  Returns what was added."""
    added = []
    from transformers.models.llama import modeling_llama as ml

    for name, obj in (("LlamaFlashAttention2", LlamaFlashAttention2), ("LlamaSdpaAttention", LlamaSdpaAttention)):
        if not hasattr(ml, name):
            setattr(ml, name, obj)
            added.append(f"modeling_llama.{name}")
    import transformers.pytorch_utils as pu

    for name, obj in (("find_pruneable_heads_and_indices", _find_pruneable_heads_and_indices),
                      ("prune_conv1d_layer", _prune_conv1d_layer)):
        if not hasattr(pu, name):
            setattr(pu, name, obj)
            added.append(f"pytorch_utils.{name}")
    try:
        import transformers.activations as act

        for name in ("silu", "gelu_new"):
            if not hasattr(act, name):
                setattr(act, name, act.ACT2FN[name])
                added.append(f"activations.{name}")
    except Exception:       # noqa: BLE001
        pass
    return added


def patch_tables(gpu_key: str = "b200") -> None:
    """Run-time rows for this GPU in the reference's peak-FLOPs and usable-memory tables, so its
    summary printer does not raise a KeyError.  2250 TFLOP/s is the dense bf16/fp16 figure."""
    import utils.train_utils as tu

    tu.GPU_TFLOPs.setdefault("bfloat16", dict(tu.GPU_TFLOPs.get("float16", {})))
    for row in ("float16", "bfloat16"):
        tu.GPU_TFLOPs[row].setdefault(gpu_key, 2250)
    tu.GPU_TFLOPs["float32"].setdefault(gpu_key, 80)
    try:
        import utils.runtime_estimator as re_

        re_.GPU_MEMORY.setdefault(gpu_key, 178.0)
    except Exception:       # noqa: BLE001
        pass
