"""Model building blocks with explicit forward and backward passes.

A `Layer` is the granule the ZeRO engine shards and the pipeline schedules execute: one
transformer block, the embedding, or the output head (the reference wraps exactly these
in one FSDP flat parameter each, zorse_utils/pipeline.py:131-148).  A layer owns no
storage: the engine binds views of its unit's flat parameter buffer (`self.p`) and flat
gradient bucket (`self.g`) before calling it.  `forward` saves what `backward` needs in a
caller-provided dict, so a schedule chooses between keeping activations and recomputing.

All math goes through an ops backend (`ops/api.py`): `sm100` kernels or the PyTorch
oracle.  Tensors are `[tokens, features]`; `ctx["B"]`, `ctx["S"]` give the microbatch
geometry.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

ALIGN = 64  # elements; every parameter starts on a 128-byte boundary of the bf16 buffer


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    init: str = "normal"  # normal | ones | zeros
    std: float = 0.02

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class Layer:
    kind = "layer"

    def __init__(self):
        self.p: dict[str, torch.Tensor] = {}
        self.g: dict[str, torch.Tensor] = {}
        self._bound_p = self._bound_g = None      # flat buffers the views in p / g were cut from
        self._layout_cache = None

    # -- parameters ---------------------------------------------------------------
    def param_specs(self) -> list[ParamSpec]:
        raise NotImplementedError

    def layout(self) -> tuple[dict[str, tuple[int, tuple]], int]:
        """name -> (offset, shape) inside the flat buffer, and the total (unpadded) length."""
        if self._layout_cache is None:
            off, out = 0, {}
            for s in self.param_specs():
                out[s.name] = (off, s.shape)
                off += (s.numel + ALIGN - 1) // ALIGN * ALIGN
            self._layout_cache = (out, off)
        return self._layout_cache

    def num_params(self) -> int:
        return sum(s.numel for s in self.param_specs())

    def bind(self, flat_params: Optional[torch.Tensor], flat_grads: Optional[torch.Tensor]) -> None:
        """Cuts the per-parameter views out of the flat buffers. Schedules call this for every
        (layer, microbatch); the views are rebuilt only when a different buffer object arrives."""
        lay, _ = self.layout()
        if flat_params is not self._bound_p:
            self.p = ({} if flat_params is None else
                      {n: flat_params[o:o + math.prod(sh)].view(sh) for n, (o, sh) in lay.items()})
            self._bound_p = flat_params
        if flat_grads is not self._bound_g:
            self.g = ({} if flat_grads is None else
                      {n: flat_grads[o:o + math.prod(sh)].view(sh) for n, (o, sh) in lay.items()})
            self._bound_g = flat_grads

    def init_flat(self, flat: torch.Tensor, seed: int) -> None:
        """Fills `flat` (any float dtype) deterministically from `seed` with a generator on
        flat's own device: the same seed gives the same tensor on every rank of a job, whatever
        the sharding or stage split (CPU and CUDA generators give different streams)."""
        lay, total = self.layout()
        flat.zero_()
        dev = flat.device
        gen = torch.Generator(device=dev).manual_seed(seed)
        for s in self.param_specs():
            o, sh = lay[s.name]
            dst = flat[o:o + s.numel]
            if s.init == "normal":
                if dst.dtype == torch.float32:
                    dst.normal_(0.0, s.std, generator=gen)
                else:
                    dst.copy_(torch.empty(s.numel, dtype=torch.float32, device=dev).normal_(0.0, s.std, generator=gen))
            elif s.init == "ones":
                dst.fill_(1.0)

    # -- compute ------------------------------------------------------------------
    def forward(self, x, ctx: dict, ops, saved: Optional[dict]):
        raise NotImplementedError

    def backward(self, dy, ctx: dict, ops, saved: dict):
        raise NotImplementedError

    def flops_per_token(self, S: int) -> float:
        return 2.0 * self.num_params()


def _norm(ops, kind, x, w, b, eps):
    return ops.norm_fwd(x, w, b if kind == "ln" else None, eps, kind == "ln")


class TransformerBlock(Layer):
    """Generic block: {RMSNorm|LayerNorm} x {pre|post}-norm x {SwiGLU|GELU|ReLU} MLP x
    {RoPE|none} x {causal|bidirectional} x optional sliding window, MHA or GQA.

    Llama/Mistral: rms, pre, swiglu, rope, causal (reference models/llama_simple.py:391-518,
    models/mistral_simple.py:20); OPT/GPT: ln, pre or post, gelu/relu, biases, learned
    positions in the embedding (models/gpt_simple.py:16-160); BERT: ln, post, erf-GELU
    (models/bert_simple.py:15-491); ViT: ln, pre, bidirectional (models/vit_simple.py:14-368).
    """
    kind = "block"

    def __init__(self, hidden: int, heads: int, kv_heads: int, ffn: int, *, norm: str = "rms", pre_norm: bool = True,
                 act: str = "swiglu", bias: bool = False, rope_theta: Optional[float] = 10000.0, causal: bool = True,
                 window: int = 0, eps: float = 1e-5, head_dim: Optional[int] = None, init_std: float = 0.02):
        super().__init__()
        self.H, self.Hq, self.Hkv, self.F = hidden, heads, kv_heads, ffn
        self.D = head_dim or hidden // heads
        self.norm, self.pre_norm, self.act, self.bias = norm, pre_norm, act, bias
        self.rope_theta, self.causal, self.window, self.eps = rope_theta, causal, window, eps
        self.std = init_std
        self._cs = None

    def param_specs(self):
        H, D, F = self.H, self.D, self.F
        qkv_w = (self.Hq + 2 * self.Hkv) * D
        sp = [ParamSpec("norm1_w", (H,), "ones")]
        if self.norm == "ln":
            sp.append(ParamSpec("norm1_b", (H,), "zeros"))
        sp.append(ParamSpec("qkv_w", (qkv_w, H), std=self.std))
        if self.bias:
            sp.append(ParamSpec("qkv_b", (qkv_w,), "zeros"))
        sp.append(ParamSpec("o_w", (H, self.Hq * D), std=self.std))
        if self.bias:
            sp.append(ParamSpec("o_b", (H,), "zeros"))
        sp.append(ParamSpec("norm2_w", (H,), "ones"))
        if self.norm == "ln":
            sp.append(ParamSpec("norm2_b", (H,), "zeros"))
        up = 2 * F if self.act == "swiglu" else F
        sp.append(ParamSpec("up_w", (up, H), std=self.std))
        if self.bias:
            sp.append(ParamSpec("up_b", (up,), "zeros"))
        sp.append(ParamSpec("down_w", (H, F), std=self.std))
        if self.bias:
            sp.append(ParamSpec("down_b", (H,), "zeros"))
        return sp

    def _rope(self, ops, S, device):
        if self.rope_theta is None:
            return None
        if self._cs is None or self._cs.shape[0] < S or self._cs.device != torch.device(device):
            self._cs = ops.rope_table(S, self.D, self.rope_theta, device)
        return self._cs

    # ---- sub-blocks ---------------------------------------------------------------
    def _attn_fwd(self, xin, resid, ctx, ops, sv):
        p, B, S = self.p, ctx["B"], ctx["S"]
        ag = self.__dict__.pop("_ag", None)  # left by a fused ZeRO unit: gather the unit inside this GEMM
        if ag is not None:
            qkv = ops.linear_fwd_gather(xin, "qkv_w", ag, p.get("qkv_b"))
        else:
            qkv = ops.linear_fwd(xin, p["qkv_w"], p.get("qkv_b"))
        cs = self._rope(ops, S, xin.device)
        if cs is not None:
            ops.rope_(qkv, cs, S, self.Hq + self.Hkv, self.D)
        att, lse = ops.attn_fwd(qkv, B, S, self.Hq, self.Hkv, self.D, self.causal, self.window)
        out = ops.linear_fwd(att, p["o_w"], p.get("o_b"), addend=resid)
        if sv is not None:
            sv.update(qkv=qkv, att=att, lse=lse)
        return out

    def _attn_bwd(self, dout, xin, ctx, ops, sv, dres):
        """dout: grad of the o-projection output; returns grad wrt xin (+ dres)."""
        p, g, B, S = self.p, self.g, ctx["B"], ctx["S"]
        datt = ops.linear_dgrad(dout, p["o_w"])
        ops.linear_wgrad(dout, sv["att"], g["o_w"], g.get("o_b"))
        dqkv = ops.attn_bwd(datt, sv["qkv"], sv["att"], sv["lse"], B, S, self.Hq, self.Hkv, self.D, self.causal,
                            self.window)
        cs = self._rope(ops, S, dout.device)
        if cs is not None:
            ops.rope_(dqkv, cs, S, self.Hq + self.Hkv, self.D, backward=True)
        dxin = ops.linear_dgrad(dqkv, p["qkv_w"], addend=dres)
        ops.linear_wgrad(dqkv, xin, g["qkv_w"], g.get("qkv_b"))
        return dxin

    def _mlp_fwd(self, xin, resid, ops, sv):
        p = self.p
        hpre = ops.linear_fwd(xin, p["up_w"], p.get("up_b"))
        a = ops.swiglu_fwd(hpre) if self.act == "swiglu" else ops.act_fwd(hpre, self.act)
        out = ops.linear_fwd(a, p["down_w"], p.get("down_b"), addend=resid)
        if sv is not None:
            sv.update(hpre=hpre, mlp_a=a)
        return out

    def _mlp_bwd(self, dout, xin, ops, sv, dres):
        p, g = self.p, self.g
        da = ops.linear_dgrad(dout, p["down_w"])
        ops.linear_wgrad(dout, sv["mlp_a"], g["down_w"], g.get("down_b"))
        dh = ops.swiglu_bwd(sv["hpre"], da) if self.act == "swiglu" else ops.act_bwd(sv["hpre"], da, self.act)
        dxin = ops.linear_dgrad(dh, p["up_w"], addend=dres)
        ops.linear_wgrad(dh, xin, g["up_w"], g.get("up_b"))
        return dxin

    # ---- block ----------------------------------------------------------------------
    def forward(self, x, ctx, ops, saved=None):
        p, sv = self.p, saved
        if self.pre_norm:
            n1, st1 = _norm(ops, self.norm, x, p["norm1_w"], p.get("norm1_b"), self.eps)
            h1 = self._attn_fwd(n1, x, ctx, ops, sv)
            n2, st2 = _norm(ops, self.norm, h1, p["norm2_w"], p.get("norm2_b"), self.eps)
            out = self._mlp_fwd(n2, h1, ops, sv)
            if sv is not None:
                sv.update(x=x, n1=n1, st1=st1, h1=h1, n2=n2, st2=st2)
        else:
            r1 = self._attn_fwd(x, x, ctx, ops, sv)
            h1, st1 = _norm(ops, self.norm, r1, p["norm1_w"], p.get("norm1_b"), self.eps)
            r2 = self._mlp_fwd(h1, h1, ops, sv)
            out, st2 = _norm(ops, self.norm, r2, p["norm2_w"], p.get("norm2_b"), self.eps)
            if sv is not None:
                sv.update(x=x, r1=r1, st1=st1, h1=h1, r2=r2, st2=st2)
        return out

    def backward(self, dy, ctx, ops, saved):
        p, g, sv = self.p, self.g, saved
        ln = self.norm == "ln"
        if self.pre_norm:
            dn2 = self._mlp_bwd(dy, sv["n2"], ops, sv, None)
            dh1 = ops.norm_bwd(dn2, sv["h1"], p["norm2_w"], sv["st2"], dy, g["norm2_w"], g.get("norm2_b"), ln)
            dn1 = self._attn_bwd(dh1, sv["n1"], ctx, ops, sv, None)
            dx = ops.norm_bwd(dn1, sv["x"], p["norm1_w"], sv["st1"], dh1, g["norm1_w"], g.get("norm1_b"), ln)
        else:
            dr2 = ops.norm_bwd(dy, sv["r2"], p["norm2_w"], sv["st2"], None, g["norm2_w"], g.get("norm2_b"), ln)
            dh1 = self._mlp_bwd(dr2, sv["h1"], ops, sv, dr2)
            dr1 = ops.norm_bwd(dh1, sv["r1"], p["norm1_w"], sv["st1"], None, g["norm1_w"], g.get("norm1_b"), ln)
            dx = self._attn_bwd(dr1, sv["x"], ctx, ops, sv, dr1)
        return dx

    def flops_per_token(self, S):
        attn = 4.0 * S * self.Hq * self.D * (0.5 if self.causal else 1.0)
        return 2.0 * self.num_params() + attn


class EmbeddingLayer(Layer):
    """Token embedding (+ learned positions, + LayerNorm for BERT-style models)."""
    kind = "embedding"

    def __init__(self, vocab: int, hidden: int, *, max_positions: int = 0, pos_offset: int = 0, post_norm: bool = False,
                 eps: float = 1e-5, init_std: float = 0.02):
        super().__init__()
        self.V, self.H, self.max_pos, self.pos_offset = vocab, hidden, max_positions, pos_offset
        self.post_norm, self.eps, self.std = post_norm, eps, init_std

    def param_specs(self):
        sp = [ParamSpec("tok", (self.V, self.H), std=self.std)]
        if self.max_pos:
            sp.append(ParamSpec("pos", (self.max_pos + self.pos_offset, self.H), std=self.std))
        if self.post_norm:
            sp += [ParamSpec("norm_w", (self.H,), "ones"), ParamSpec("norm_b", (self.H,), "zeros")]
        return sp

    def forward(self, ids, ctx, ops, saved=None):
        S = ctx["S"]
        e = ops.embedding_fwd(ids.reshape(-1), self.p["tok"], self.p.get("pos"), S, self.pos_offset)
        if self.post_norm:
            y, st = ops.norm_fwd(e, self.p["norm_w"], self.p["norm_b"], self.eps, True)
            if saved is not None:
                saved.update(e=e, st=st)
            e = y
        if saved is not None:
            saved["ids"] = ids
        return e

    def backward(self, dy, ctx, ops, saved):
        if self.post_norm:
            dy = ops.norm_bwd(dy, saved["e"], self.p["norm_w"], saved["st"], None, self.g["norm_w"], self.g["norm_b"], True)
        ops.embedding_bwd(saved["ids"].reshape(-1), dy, self.g["tok"], self.g.get("pos"), ctx["S"], self.pos_offset)
        return None

    def flops_per_token(self, S):
        return 0.0


class PatchEmbeddingLayer(Layer):
    """ViT patch embedding: non-overlapping patches flattened and projected (a strided
    convolution written as a GEMM), plus a class token and learned positions
    (reference models/vit_simple.py:143)."""
    kind = "embedding"

    def __init__(self, image: int, patch: int, channels: int, hidden: int, init_std: float = 0.02):
        super().__init__()
        self.image, self.patch, self.C, self.H, self.std = image, patch, channels, hidden, init_std
        self.n_patches = (image // patch) ** 2
        self.kdim = (channels * patch * patch + 7) // 8 * 8

    def param_specs(self):
        return [ParamSpec("proj_w", (self.H, self.kdim), std=self.std), ParamSpec("proj_b", (self.H,), "zeros"),
                ParamSpec("cls", (1, self.H), std=self.std), ParamSpec("pos", (self.n_patches + 1, self.H), std=self.std)]

    def tokens_per_image(self):
        return self.n_patches + 1

    def _patches(self, img):
        B = img.shape[0]
        pt = torch.nn.functional.unfold(img.float(), self.patch, stride=self.patch).transpose(1, 2)
        pt = pt.reshape(B * self.n_patches, -1)
        if pt.shape[1] != self.kdim:
            pt = torch.nn.functional.pad(pt, (0, self.kdim - pt.shape[1]))
        return pt.to(self.p["proj_w"].dtype).contiguous()

    def forward(self, img, ctx, ops, saved=None):
        B = img.shape[0]
        pt = self._patches(img)
        e = ops.linear_fwd(pt, self.p["proj_w"], self.p["proj_b"]).view(B, self.n_patches, self.H)
        x = torch.cat([self.p["cls"].expand(B, 1, self.H), e], dim=1) + self.p["pos"][None]
        if saved is not None:
            saved["pt"] = pt
        return x.reshape(B * (self.n_patches + 1), self.H).contiguous()

    def backward(self, dy, ctx, ops, saved):
        B = dy.shape[0] // (self.n_patches + 1)
        d = dy.view(B, self.n_patches + 1, self.H)
        self.g["pos"].add_(d.float().sum(0).to(self.g["pos"].dtype))
        self.g["cls"].add_(d[:, 0].float().sum(0, keepdim=True).to(self.g["cls"].dtype))
        de = d[:, 1:].reshape(B * self.n_patches, self.H).contiguous()
        ops.linear_wgrad(de, saved["pt"], self.g["proj_w"], self.g["proj_b"])
        return None


class HeadLayer(Layer):
    """Final norm + output projection + cross-entropy.  `forward` returns the per-row
    losses; with `targets` in ctx, `loss_and_backward` fuses loss and the gradient wrt the
    logits so the logits tensor is written once and overwritten in place by its gradient."""
    kind = "head"

    def __init__(self, hidden: int, vocab: int, *, norm: Optional[str] = "rms", eps: float = 1e-5, pool: Optional[str] = None,
                 bias: bool = False, init_std: float = 0.02):
        super().__init__()
        self.H, self.V, self.norm, self.eps, self.pool, self.bias, self.std = hidden, vocab, norm, eps, pool, bias, init_std

    def param_specs(self):
        sp = []
        if self.norm:
            sp.append(ParamSpec("norm_w", (self.H,), "ones"))
            if self.norm == "ln":
                sp.append(ParamSpec("norm_b", (self.H,), "zeros"))
        sp.append(ParamSpec("head_w", (self.V, self.H), std=self.std))
        if self.bias:
            sp.append(ParamSpec("head_b", (self.V,), "zeros"))
        return sp

    def _pool(self, x, ctx):
        if self.pool is None:
            return x
        B, S = ctx["B"], ctx["S"]
        xv = x.view(B, S, self.H)
        return (xv[:, 0] if self.pool == "first" else xv.float().mean(1).to(x.dtype)).contiguous()

    def _unpool(self, dx, ctx, like):
        if self.pool is None:
            return dx
        B, S = ctx["B"], ctx["S"]
        out = torch.zeros(B, S, self.H, dtype=dx.dtype, device=dx.device)
        if self.pool == "first":
            out[:, 0] = dx
        else:
            out += (dx.float() / S).to(dx.dtype)[:, None, :]
        return out.view(B * S, self.H)

    def logits(self, x, ctx, ops, saved=None):
        xp = self._pool(x, ctx)
        if self.norm:
            n, st = _norm(ops, self.norm, xp, self.p["norm_w"], self.p.get("norm_b"), self.eps)
        else:
            n, st = xp, None
        if saved is not None:
            saved.update(xp=xp, n=n, st=st)
        ag = self.__dict__.pop("_ag", None)
        if ag is not None:
            return ops.linear_fwd_gather(n, "head_w", ag, self.p.get("head_b"))
        return ops.linear_fwd(n, self.p["head_w"], self.p.get("head_b"))

    def forward(self, x, ctx, ops, saved=None):
        lg = self.logits(x, ctx, ops, saved)
        rows, dlg = ops.cross_entropy(lg, ctx["targets"].reshape(-1), ctx.get("loss_scale", 1.0),
                                      want_grad=saved is not None)
        if saved is not None:
            saved["dlogits"] = dlg
        return rows

    def backward(self, dy, ctx, ops, saved):
        """dy is ignored: the loss gradient was produced by forward (scaled by ctx['loss_scale'])."""
        dlg = saved["dlogits"]
        dn = ops.linear_dgrad(dlg, self.p["head_w"])
        ops.linear_wgrad(dlg, saved["n"], self.g["head_w"], self.g.get("head_b"))
        if self.norm:
            dxp = ops.norm_bwd(dn, saved["xp"], self.p["norm_w"], saved["st"], None, self.g["norm_w"],
                               self.g.get("norm_b"), self.norm == "ln")
        else:
            dxp = dn
        return self._unpool(dxp, ctx, saved["xp"])

    def flops_per_token(self, S):
        return 2.0 * self.V * self.H


class NoOpLayer(Layer):
    """Identity with one dummy parameter (placeholder unit; reference models/common.py:6-15)."""
    kind = "noop"

    def param_specs(self):
        return [ParamSpec("dummy", (ALIGN,), "zeros")]

    def forward(self, x, ctx, ops, saved=None):
        return x

    def backward(self, dy, ctx, ops, saved):
        return dy
