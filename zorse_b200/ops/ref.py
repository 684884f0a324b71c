"""Pure-PyTorch restatement of every op (runs on CPU, any dtype).

This is the oracle the sm_100a kernels are tested against and the compute backend of the
CPU/gloo configuration.  Shapes follow the packed layouts the CUDA kernels use:
`qkv` is `[T, (Hq + 2*Hkv) * D]` (query heads, key heads, value heads).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ w.t()
    return y if b is None else y + b


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype)


def layernorm(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    xf = x.float()
    mu = xf.mean(-1, keepdim=True)
    var = (xf - mu).pow(2).mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(var + eps) * w.float()
    if b is not None:
        y = y + b.float()
    return y.to(x.dtype)


def rope_table(S: int, d: int, theta: float, device=None) -> torch.Tensor:
    """[S, d] fp32: cos (d/2) | sin (d/2) for positions 0..S-1 (rotate-half convention)."""
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=device) / d))
    ang = torch.arange(S, dtype=torch.float64, device=device)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1).float()


def rope(qkv: torch.Tensor, cs: torch.Tensor, S: int, nheads: int, d: int, backward: bool = False) -> torch.Tensor:
    """Rotates heads [0, nheads) of packed qkv [T, width]; returns a new tensor."""
    T = qkv.shape[0]
    out = qkv.clone()
    x = qkv[:, : nheads * d].float().reshape(T, nheads, d)
    pos = torch.arange(T, device=qkv.device) % S
    cos = cs[pos, : d // 2][:, None, :]
    sin = cs[pos, d // 2:][:, None, :]
    if backward:
        sin = -sin
    a, b = x[..., : d // 2], x[..., d // 2:]
    y = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    out[:, : nheads * d] = y.reshape(T, nheads * d).to(qkv.dtype)
    return out


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    F_ = gu.shape[-1] // 2
    g, u = gu[..., :F_].float(), gu[..., F_:].float()
    return (F.silu(g) * u).to(gu.dtype)


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    xf = x.float()
    if kind == "relu":
        y = F.relu(xf)
    elif kind == "gelu_erf":
        y = F.gelu(xf)
    else:
        y = F.gelu(xf, approximate="tanh")
    return y.to(x.dtype)


def attention(qkv: torch.Tensor, B: int, S: int, Hq: int, Hkv: int, D: int, causal: bool = True,
              window: int = 0, scale: Optional[float] = None) -> torch.Tensor:
    """Explicit masked-softmax attention in fp32. Returns [B*S, Hq*D] in qkv's dtype."""
    sc = 1.0 / math.sqrt(D) if scale is None else scale
    x = qkv.float().reshape(B, S, Hq + 2 * Hkv, D)
    q = x[:, :, :Hq].permute(0, 2, 1, 3)
    k = x[:, :, Hq:Hq + Hkv].permute(0, 2, 1, 3)
    v = x[:, :, Hq + Hkv:].permute(0, 2, 1, 3)
    rep = Hq // Hkv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    s = (q @ k.transpose(-1, -2)) * sc
    i = torch.arange(S, device=qkv.device)[:, None]
    j = torch.arange(S, device=qkv.device)[None, :]
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device)
    if causal:
        mask &= j <= i
    if window and window > 0:
        mask &= (i - j) < window
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = p @ v
    return o.permute(0, 2, 1, 3).reshape(B * S, Hq * D).to(qkv.dtype)


def cross_entropy_rows(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    return F.cross_entropy(logits.float(), targets, reduction="none")


def embedding(ids: torch.Tensor, table: torch.Tensor, pos_table: Optional[torch.Tensor] = None, S: int = 1,
              pos_offset: int = 0) -> torch.Tensor:
    out = table[ids.reshape(-1)]
    if pos_table is not None:
        pos = torch.arange(ids.numel(), device=ids.device) % S + pos_offset
        out = out + pos_table[pos]
    return out


def adam_step(p, m, v, g, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    """In-place fp32 Adam with torch.optim.Adam arithmetic."""
    g = g.float() * grad_scale
    if weight_decay:
        g = g + weight_decay * p
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = v.sqrt() / math.sqrt(bc2) + eps
    p.addcdiv_(m, denom, value=-lr / bc1)
