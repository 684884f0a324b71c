"""Tensor-parallel layers with sequence-parallel activations.

The tp processes of a lane each hold a slice of every transformer block: whole attention heads
(query heads and their key/value heads) and a 1/tp slice of the MLP width.  Activations between
sub-blocks are split by rows (tokens): every process keeps `tokens / tp` rows, normalises them,
and the rows are all-gathered in front of the column-split GEMMs (QKV, gate/up) and
reduce-scattered behind the row-split ones (attention output, down projection), so the two
collectives per sub-block move what one all-reduce would and the norms, residual adds and
stage-to-stage messages shrink by tp.  The embedding and the head are not split: each process
embeds / scores its own rows with the full table (vocabulary projection and loss over 1/tp of
the tokens, no communication), and their gradients — like those of the norm weights and of the
biases added behind a reduce-scatter — are summed over the lane before the data-parallel
reduction (`tp_replicated_ranges`).

The reference carries this idea only as an unused DTensor plan (column-/row-wise linears with
sequence-parallel norms, models/parallelize_model.py:107-173); here it is part of the layer
classes with explicit forward and backward, like everything else.

Initial values equal those of the unsplit model: `init_flat` draws every full parameter with the
unsplit layer's generator sequence and keeps this process's slice.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from .layers import EmbeddingLayer, HeadLayer, Layer, TransformerBlock, _norm


class TPComm:
    """The lane's collectives on row-split activations (NCCL on GPUs, gloo on CPU ranks)."""

    def __init__(self, pg, size: int, index: int):
        self.pg, self.size, self.index = pg, size, index

    def gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty((x.shape[0] * self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.pg)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty((x.shape[0] // self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=self.pg)
        return out

    def linear_rs(self, ops, x: torch.Tensor, w: torch.Tensor, w_kmajor: bool, resid=None, bias=None) -> torch.Tensor:
        """Rows of sum over the lane of `x @ w^T` (w_kmajor, a forward projection with w [out, in]) or
        `x @ w` (an input gradient with w [in, out]), plus residual rows and bias: a row-split GEMM and
        the reduce-scatter behind it.  Here: library GEMM call + library collective + ATen adds;
        `parallel/tp_fused.py` replaces the three by two kernels."""
        part = ops.linear_fwd(x, w, None) if w_kmajor else ops.linear_dgrad(x, w)
        out = self.reduce_scatter_rows(part)
        if resid is not None:
            out += resid
        if bias is not None:
            out += bias
        return out

    def norm_gather(self, ops, x, w, b, eps: float, kind: str):
        """Norm of this process's rows and the lane's gathered result: (rows, stats, all rows).  The gathered
        tensor is only valid until the next gather (the fused lane hands out a staging buffer)."""
        n, st = _norm(ops, kind, x, w, b, eps)
        return n, st, self.gather_rows(n)

    def linear_rs_norm_gather(self, ops, x, wmat, w_kmajor: bool, resid, bias, w, b, eps: float, kind: str):
        """linear_rs followed by norm_gather of its result: (sum rows, normalised rows, stats, all normalised rows)."""
        h = self.linear_rs(ops, x, wmat, w_kmajor, resid, bias)
        n, st, nf = self.norm_gather(ops, h, w, b, eps, kind)
        return h, n, st, nf

    def rows(self, n: int) -> tuple[int, int]:
        """This process's [lo, hi) of n rows."""
        if n % self.size:
            raise ValueError(f"{n} rows do not split over {self.size} tensor-parallel processes")
        k = n // self.size
        return self.index * k, (self.index + 1) * k


def take_slice(full: torch.Tensor, dim: int, segments: tuple[int, ...], tp: int, index: int) -> torch.Tensor:
    """`full` is a concatenation of `segments` along `dim`; returns the concatenation of part
    `index` (of tp equal parts) of every segment."""
    parts = torch.split(full, list(segments), dim=dim)
    return torch.cat([torch.chunk(p, tp, dim=dim)[index] for p in parts], dim=dim).contiguous()


def put_slice(full: torch.Tensor, piece: torch.Tensor, dim: int, segments: tuple[int, ...], tp: int, index: int) -> None:
    """Inverse of take_slice for one process: writes `piece` into its places of `full`."""
    at = 0
    for seg, src in zip(segments, torch.split(piece, [s // tp for s in segments], dim=dim)):
        k = seg // tp
        full.narrow(dim, at + index * k, k).copy_(src)
        at += seg


class TPTransformerBlock(TransformerBlock):
    """Slice `tp_index` of a transformer block (pre- or post-norm) split over `tp` processes."""

    def __init__(self, hidden: int, heads: int, kv_heads: int, ffn: int, *, tp: int, tp_index: int, **kw):
        if heads % tp or kv_heads % tp or ffn % tp:
            raise ValueError(f"tensor parallelism {tp} must divide heads {heads}, kv heads {kv_heads} and ffn {ffn}")
        self.whole = TransformerBlock(hidden, heads, kv_heads, ffn, **kw)
        super().__init__(hidden, heads // tp, kv_heads // tp, ffn // tp, head_dim=self.whole.D,
                         **{k: v for k, v in kw.items() if k != "head_dim"})
        self.tp, self.tp_index = tp, tp_index

    # how each parameter of the unsplit block is cut: name -> (dim, segments along that dim)
    def _cuts(self) -> dict:
        w = self.whole
        qkv = (w.Hq * w.D, w.Hkv * w.D, w.Hkv * w.D)
        up = (w.F, w.F) if w.act == "swiglu" else (w.F,)
        return {"qkv_w": (0, qkv), "qkv_b": (0, qkv), "o_w": (1, (w.Hq * w.D,)), "up_w": (0, up), "up_b": (0, up),
                "down_w": (1, (w.F,))}

    def init_flat(self, flat: torch.Tensor, seed: int) -> None:
        wl, wn = self.whole.layout()
        tmp = torch.empty(wn, dtype=torch.float32, device=flat.device)
        self.whole.init_flat(tmp, seed)
        self.load_from_whole(flat, tmp)

    def load_from_whole(self, flat: torch.Tensor, whole_flat: torch.Tensor) -> None:
        """Fills this slice's flat buffer from the unsplit block's flat buffer."""
        wl, _ = self.whole.layout()
        lay, _ = self.layout()
        cuts = self._cuts()
        flat.zero_()
        for name, (o, sh) in lay.items():
            wo, wsh = wl[name]
            src = whole_flat[wo:wo + math.prod(wsh)].view(wsh)
            if name in cuts:
                dim, seg = cuts[name]
                src = take_slice(src, dim, seg, self.tp, self.tp_index)
            flat[o:o + math.prod(sh)].copy_(src.reshape(-1))

    def store_into_whole(self, flat: torch.Tensor, whole_flat: torch.Tensor) -> None:
        """Writes this slice's parameters into their places of the unsplit block's flat buffer
        (replicated parameters are simply copied)."""
        wl, _ = self.whole.layout()
        lay, _ = self.layout()
        cuts = self._cuts()
        for name, (o, sh) in lay.items():
            wo, wsh = wl[name]
            dst = whole_flat[wo:wo + math.prod(wsh)].view(wsh)
            piece = flat[o:o + math.prod(sh)].view(sh)
            if name in cuts:
                dim, seg = cuts[name]
                put_slice(dst, piece, dim, seg, self.tp, self.tp_index)
            else:
                dst.copy_(piece)

    def tp_replicated_ranges(self) -> list[tuple[int, int]]:
        lay, _ = self.layout()
        cuts = self._cuts()
        return [(o, math.prod(sh)) for name, (o, sh) in lay.items() if name not in cuts]

    # ---- sub-blocks: rows in, rows out -----------------------------------------------------
    # The gradient of a reduce-scatter is an all-gather and the other way round.
    def _attn_core_fwd(self, xin_all, ctx, ops, sv):
        """Gathered rows in, this process's heads' attention output (all rows) out."""
        p, B, S = self.p, ctx["B"], ctx["S"]
        qkv = ops.linear_fwd(xin_all, p["qkv_w"], p.get("qkv_b"))
        cs = self._rope(ops, S, xin_all.device)
        if cs is not None:
            ops.rope_(qkv, cs, S, self.Hq + self.Hkv, self.D)
        att, lse = ops.attn_fwd(qkv, B, S, self.Hq, self.Hkv, self.D, self.causal, self.window)
        if sv is not None:
            sv.update(qkv=qkv, att=att, lse=lse)
        return att

    def _mlp_core_fwd(self, xin_all, ops, sv):
        p = self.p
        hpre = ops.linear_fwd(xin_all, p["up_w"], p.get("up_b"))
        a = ops.swiglu_fwd(hpre) if self.act == "swiglu" else ops.act_fwd(hpre, self.act)
        if sv is not None:
            sv.update(hpre=hpre, mlp_a=a)
        return a

    def _attn_rows_bwd(self, dout, xin, ctx, ops, sv):
        """dout: gradient of the sub-block's output rows; returns the gradient reaching xin through the
        projections (the residual branch is added by the caller)."""
        p, g, tp, B, S = self.p, self.g, ctx["tp"], ctx["B"], ctx["S"]
        if "o_b" in g:
            g["o_b"].add_(dout.float().sum(0).to(g["o_b"].dtype))
        df = tp.gather_rows(dout)
        datt = ops.linear_dgrad(df, p["o_w"])
        ops.linear_wgrad(df, sv["att"], g["o_w"], None)
        dqkv = ops.attn_bwd(datt, sv["qkv"], sv["att"], sv["lse"], B, S, self.Hq, self.Hkv, self.D, self.causal,
                            self.window)
        cs = self._rope(ops, S, dout.device)
        if cs is not None:
            ops.rope_(dqkv, cs, S, self.Hq + self.Hkv, self.D, backward=True)
        dxin = tp.linear_rs(ops, dqkv, p["qkv_w"], False)
        ops.linear_wgrad(dqkv, tp.gather_rows(xin), g["qkv_w"], g.get("qkv_b"))
        return dxin

    def _mlp_rows_bwd(self, dout, xin, ctx, ops, sv):
        p, g, tp = self.p, self.g, ctx["tp"]
        if "down_b" in g:
            g["down_b"].add_(dout.float().sum(0).to(g["down_b"].dtype))
        df = tp.gather_rows(dout)
        da = ops.linear_dgrad(df, p["down_w"])
        ops.linear_wgrad(df, sv["mlp_a"], g["down_w"], None)
        dh = ops.swiglu_bwd(sv["hpre"], da) if self.act == "swiglu" else ops.act_bwd(sv["hpre"], da, self.act)
        dxin = tp.linear_rs(ops, dh, p["up_w"], False)
        ops.linear_wgrad(dh, tp.gather_rows(xin), g["up_w"], g.get("up_b"))
        return dxin

    # ---- block ------------------------------------------------------------------------------
    def forward(self, x, ctx, ops, saved=None):
        p, sv, tp, kind, eps = self.p, saved, ctx["tp"], self.norm, self.eps
        if self.pre_norm:
            n1, st1, n1_all = tp.norm_gather(ops, x, p["norm1_w"], p.get("norm1_b"), eps, kind)
            att = self._attn_core_fwd(n1_all, ctx, ops, sv)
            h1, n2, st2, n2_all = tp.linear_rs_norm_gather(ops, att, p["o_w"], True, x, p.get("o_b"),
                                                           p["norm2_w"], p.get("norm2_b"), eps, kind)
            a = self._mlp_core_fwd(n2_all, ops, sv)
            out = tp.linear_rs(ops, a, p["down_w"], True, h1, p.get("down_b"))
            if sv is not None:
                sv.update(x=x, n1=n1, st1=st1, h1=h1, n2=n2, st2=st2)
        else:
            att = self._attn_core_fwd(tp.gather_rows(x), ctx, ops, sv)
            r1, h1, st1, h1_all = tp.linear_rs_norm_gather(ops, att, p["o_w"], True, x, p.get("o_b"),
                                                           p["norm1_w"], p.get("norm1_b"), eps, kind)
            a = self._mlp_core_fwd(h1_all, ops, sv)
            r2 = tp.linear_rs(ops, a, p["down_w"], True, h1, p.get("down_b"))
            out, st2 = _norm(ops, kind, r2, p["norm2_w"], p.get("norm2_b"), eps)
            if sv is not None:
                sv.update(x=x, r1=r1, st1=st1, h1=h1, r2=r2, st2=st2)
        return out

    def backward(self, dy, ctx, ops, saved):
        p, g, sv = self.p, self.g, saved
        ln = self.norm == "ln"
        if self.pre_norm:
            dn2 = self._mlp_rows_bwd(dy, sv["n2"], ctx, ops, sv)
            dh1 = ops.norm_bwd(dn2, sv["h1"], p["norm2_w"], sv["st2"], dy, g["norm2_w"], g.get("norm2_b"), ln)
            dn1 = self._attn_rows_bwd(dh1, sv["n1"], ctx, ops, sv)
            return ops.norm_bwd(dn1, sv["x"], p["norm1_w"], sv["st1"], dh1, g["norm1_w"], g.get("norm1_b"), ln)
        dr2 = ops.norm_bwd(dy, sv["r2"], p["norm2_w"], sv["st2"], None, g["norm2_w"], g.get("norm2_b"), ln)
        dh1 = self._mlp_rows_bwd(dr2, sv["h1"], ctx, ops, sv)
        dh1 += dr2
        dr1 = ops.norm_bwd(dh1, sv["r1"], p["norm1_w"], sv["st1"], None, g["norm1_w"], g.get("norm1_b"), ln)
        dx = self._attn_rows_bwd(dr1, sv["x"], ctx, ops, sv)
        dx += dr1
        return dx


class _RowSplit:
    """Mixin of the two unsplit layers: every process works on its own rows with the full weights."""
    tp = 1
    tp_index = 0

    def tp_replicated_ranges(self) -> list[tuple[int, int]]:
        return [(0, self.layout()[1])]


class SPEmbeddingLayer(_RowSplit, EmbeddingLayer):
    def __init__(self, *a, tp: int, tp_index: int, **kw):
        super().__init__(*a, **kw)
        self.tp, self.tp_index = tp, tp_index

    def forward(self, ids, ctx, ops, saved=None):
        e = super().forward(ids, ctx, ops, saved)
        lo, hi = ctx["tp"].rows(e.shape[0])
        return e[lo:hi].contiguous()

    def backward(self, dy, ctx, ops, saved):
        # positions and the optional norm are row-wise: run the unsplit backward on a gradient that
        # is zero outside this process's rows
        T = dy.shape[0] * self.tp
        lo, hi = ctx["tp"].rows(T)
        full = torch.zeros((T,) + tuple(dy.shape[1:]), dtype=dy.dtype, device=dy.device)
        full[lo:hi] = dy       # a zero row adds nothing to the table, position or norm gradients
        return super().backward(full, ctx, ops, saved)


class SPHeadLayer(_RowSplit, HeadLayer):
    def __init__(self, *a, tp: int, tp_index: int, **kw):
        super().__init__(*a, **kw)
        if self.pool:
            raise NotImplementedError("tensor parallelism does not cover pooled (classification) heads")
        self.tp, self.tp_index = tp, tp_index

    def forward(self, x, ctx, ops, saved=None):
        t = ctx["targets"].reshape(-1)
        lo, hi = ctx["tp"].rows(t.shape[0])
        return super().forward(x, dict(ctx, targets=t[lo:hi]), ops, saved)


def replicated_ranges(layer: Layer) -> list[tuple[int, int]]:
    fn = getattr(layer, "tp_replicated_ranges", None)
    return fn() if fn is not None else []
