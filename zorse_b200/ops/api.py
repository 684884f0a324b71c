"""Op layer: one interface, two backends.

* `Sm100Ops` – the product path: every method launches hand-written sm_100a kernels
  (`ops/sm100.py`); bf16 activations/weights, fp32 or bf16 gradient buckets.
* `RefOps`   – pure PyTorch (`ops/ref.py`); runs on CPU in any dtype.  It is the test
  oracle and the compute path of the CPU/gloo configuration.

Models call forward *and* backward ops explicitly (no autograd): weight gradients are
accumulated straight into views of the ZeRO unit's flat gradient bucket.  All tensors
are 2-D `[tokens, features]`.
"""
from __future__ import annotations

import torch

from . import ref

_ACT_KINDS = {"gelu": 0, "gelu_new": 0, "gelu_tanh": 0, "relu": 1, "gelu_erf": 2}


class RefOps:
    name = "ref"

    # ---- linear -----------------------------------------------------------------
    def linear_fwd(self, x, w, bias=None, addend=None):
        y = x @ w.t()
        if bias is not None:
            y = y + bias
        if addend is not None:
            y = y + addend
        return y

    def linear_dgrad(self, dy, w, addend=None):
        dx = dy @ w
        return dx if addend is None else dx + addend

    def linear_wgrad(self, dy, x, gw, gb=None):
        gw.add_((dy.float().t() @ x.float()).to(gw.dtype))
        if gb is not None:
            gb.add_(dy.float().sum(0).to(gb.dtype))

    # ---- norms ------------------------------------------------------------------
    def norm_fwd(self, x, w, b, eps, ln):
        xf = x.float()
        mean = xf.mean(-1) if ln else torch.zeros(x.shape[0], device=x.device)
        var = (xf - mean[:, None]).pow(2).mean(-1)
        rstd = torch.rsqrt(var + eps)
        y = (xf - mean[:, None]) * rstd[:, None] * w.float()
        if ln and b is not None:
            y = y + b.float()
        return y.to(x.dtype), torch.stack([mean, rstd], dim=1)

    def norm_bwd(self, dy, x, w, stats, dres, gw, gb, ln):
        xf, dyf = x.float(), dy.float()
        mean, rstd = stats[:, 0:1], stats[:, 1:2]
        xh = (xf - mean) * rstd
        g = dyf * w.float()
        m1 = (g * xh).mean(-1, keepdim=True)
        m2 = g.mean(-1, keepdim=True) if ln else 0.0
        dx = rstd * (g - xh * m1 - m2)
        if dres is not None:
            dx = dx + dres.float()
        if gw is not None:
            gw.add_((dyf * xh).sum(0).to(gw.dtype))
        if ln and gb is not None:
            gb.add_(dyf.sum(0).to(gb.dtype))
        return dx.to(x.dtype)

    # ---- rope / attention -------------------------------------------------------
    def rope_table(self, S, d, theta, device):
        return ref.rope_table(S, d, theta, device)

    def rope_(self, qkv, cs, S, nheads, d, backward=False):
        qkv.copy_(ref.rope(qkv, cs, S, nheads, d, backward))
        return qkv

    def attn_fwd(self, qkv, B, S, Hq, Hkv, D, causal=True, window=0):
        return ref.attention(qkv, B, S, Hq, Hkv, D, causal, window), None

    def attn_bwd(self, do, qkv, o, lse, B, S, Hq, Hkv, D, causal=True, window=0):
        with torch.enable_grad():
            q = qkv.detach().float().requires_grad_(True)
            out = ref.attention(q, B, S, Hq, Hkv, D, causal, window)
            (dq,) = torch.autograd.grad(out, q, do.float())
        return dq.to(qkv.dtype)

    # ---- MLP activations --------------------------------------------------------
    def swiglu_fwd(self, gu):
        return ref.swiglu(gu)

    def swiglu_bwd(self, gu, dout):
        F_ = gu.shape[-1] // 2
        g, u, d = gu[:, :F_].float(), gu[:, F_:].float(), dout.float()
        sg = torch.sigmoid(g)
        dg = d * u * (sg * (1 + g * (1 - sg)))
        du = d * g * sg
        return torch.cat([dg, du], dim=-1).to(gu.dtype)

    def act_fwd(self, x, kind):
        return ref.activation(x, {0: "gelu", 1: "relu", 2: "gelu_erf"}[_ACT_KINDS[kind]])

    def act_bwd(self, x, dy, kind):
        with torch.enable_grad():
            xf = x.detach().float().requires_grad_(True)
            y = ref.activation(xf, {0: "gelu", 1: "relu", 2: "gelu_erf"}[_ACT_KINDS[kind]])
            (dx,) = torch.autograd.grad(y, xf, dy.float())
        return dx.to(x.dtype)

    # ---- embedding / loss / optimizer ------------------------------------------
    def embedding_fwd(self, ids, table, pos_table=None, S=1, pos_offset=0):
        return ref.embedding(ids, table, pos_table, S, pos_offset)

    def embedding_bwd(self, ids, dout, gtable, gpos=None, S=1, pos_offset=0):
        ids = ids.reshape(-1)
        gtable.index_add_(0, ids, dout.to(gtable.dtype))
        if gpos is not None:
            pos = torch.arange(ids.numel(), device=ids.device) % S + pos_offset
            gpos.index_add_(0, pos, dout.to(gpos.dtype))

    def cross_entropy(self, logits, targets, grad_scale, want_grad=True):
        lf = logits.float()
        rows = ref.cross_entropy_rows(lf, targets)
        if not want_grad:
            return rows, None
        p = torch.softmax(lf, dim=-1)
        keep = targets != -100                      # ignored positions: zero loss, zero gradient
        idx = torch.arange(lf.shape[0], device=lf.device)
        p[idx[keep], targets[keep]] -= 1.0
        p[~keep] = 0.0
        return rows, (p * grad_scale).to(logits.dtype)

    def adam_step(self, p, m, v, g, p16, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                  zero_grad=False):
        ref.adam_step(p, m, v, g, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay, step=step,
                      grad_scale=grad_scale)
        if p16 is not None:
            p16.copy_(p)
        if zero_grad:
            g.zero_()


class Sm100Ops:
    """Hand-written sm_100a kernels only. Requires bf16 CUDA tensors."""
    name = "sm100"

    def __init__(self):
        from . import sm100

        self.k = sm100
        self.k.lib()

    def linear_fwd(self, x, w, bias=None, addend=None):
        y = torch.empty(x.shape[0], w.shape[0], dtype=x.dtype, device=x.device)
        return self.k.gemm(x, w, y, bias=bias, addend=addend)

    def linear_fwd_gather(self, x, name, ag, bias=None):
        """Forward GEMM that also all-gathers the unit's parameters (see engine/fused.py)."""
        off, shape = ag.layout[name]
        y = torch.empty(x.shape[0], shape[0], dtype=x.dtype, device=x.device)
        return self.k.ag_gemm(x, ag.full, off, shape, y, shard_ptrs=ag.shard_ptrs, R=ag.R, r=ag.r,
                              shard_elems=ag.shard_n, chunk_bytes=ag.chunk_bytes, chunk_flags=ag.chunk_flags,
                              epoch=ag.epoch, version_flags=ag.version_flags, need_version=ag.need_version, bias=bias)

    def linear_dgrad(self, dy, w, addend=None):
        dx = torch.empty(dy.shape[0], w.shape[1], dtype=dy.dtype, device=dy.device)
        return self.k.gemm(dy, w, dx, b_mn=True, addend=addend)

    def linear_wgrad(self, dy, x, gw, gb=None):
        # gw[N,K] += dy^T[N,T] @ x[T,K]: both operands contiguous along the non-reduced dim
        self.k.gemm(dy, x, gw, a_mn=True, b_mn=True, accumulate=True)
        if gb is not None:
            self.k.colsum_accumulate(dy, gb)

    def norm_fwd(self, x, w, b, eps, ln):
        return self.k.norm_fwd(x, w, b, eps, ln)

    def norm_bwd(self, dy, x, w, stats, dres, gw, gb, ln):
        return self.k.norm_bwd(dy, x, w, stats, dres, gw, gb, ln)

    def rope_table(self, S, d, theta, device):
        return ref.rope_table(S, d, theta, device)

    def rope_(self, qkv, cs, S, nheads, d, backward=False):
        return self.k.rope_(qkv, cs, S, nheads, d, backward)

    def attn_fwd(self, qkv, B, S, Hq, Hkv, D, causal=True, window=0):
        return self.k.flash_fwd(qkv, B, S, Hq, Hkv, D, causal, window)

    def attn_bwd(self, do, qkv, o, lse, B, S, Hq, Hkv, D, causal=True, window=0):
        return self.k.flash_bwd(do, qkv, o, lse, B, S, Hq, Hkv, D, causal, window)

    def swiglu_fwd(self, gu):
        return self.k.swiglu_fwd(gu)

    def swiglu_bwd(self, gu, dout):
        return self.k.swiglu_bwd(gu, dout)

    def act_fwd(self, x, kind):
        return self.k.act_fwd(x, _ACT_KINDS[kind])

    def act_bwd(self, x, dy, kind):
        return self.k.act_bwd(x, dy, _ACT_KINDS[kind])

    def embedding_fwd(self, ids, table, pos_table=None, S=1, pos_offset=0):
        return self.k.embedding_fwd(ids.reshape(-1), table, pos_table, S, pos_offset)

    def embedding_bwd(self, ids, dout, gtable, gpos=None, S=1, pos_offset=0):
        self.k.embedding_bwd(ids.reshape(-1), dout, gtable, gpos, S, pos_offset)

    def cross_entropy(self, logits, targets, grad_scale, want_grad=True):
        rows = self.k.cross_entropy(logits, targets, grad_scale, dlogits=logits if want_grad else None)
        return rows, (logits if want_grad else None)  # gradient written in place

    def adam_step(self, p, m, v, g, p16, **kw):
        self.k.adam_step(p, m, v, g, p16, **kw)


_cache: dict[str, object] = {}


def get_ops(name: str):
    """'sm100' (CUDA kernels of this repository) or 'ref' (PyTorch; CPU oracle)."""
    if name not in _cache:
        if name == "ref":
            _cache[name] = RefOps()
        elif name == "sm100":
            _cache[name] = Sm100Ops()
        else:
            raise ValueError(f"unknown ops backend {name!r}")
    return _cache[name]


def default_ops_for(device) -> str:
    return "sm100" if torch.device(device).type == "cuda" else "ref"
