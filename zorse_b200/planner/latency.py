"""Per-layer compute latencies: profiled table first, analytic roofline as a fallback.

`data/model_latencies.json` has the reference's layout (written by the layer profiler):
    model -> gpu -> seq_len -> dtype -> [[fwd_slope, fwd_icpt], [bwd_slope, bwd_icpt], [fwd ms at b=1..n], [bwd ms at b=1..n]]
(older entries: only the two pairs).  A measured value at the requested microbatch size wins
over the linear model (reference utils/optimizer_utils.py:59-125).
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Optional

from ..models import registry
from .cluster import ModelLatencies

DATA_DIR = Path(__file__).resolve().parents[2] / "data"
# sustained dense bf16 TFLOP/s used by the analytic fallback (measured on this pool for b200)
ANALYTIC_TFLOPS = {"b200": 1100.0, "h100-nvl": 500.0, "h100": 550.0, "a100x80": 230.0, "a100": 230.0, "l40s": 180.0,
                   "a6000": 90.0, "l4": 60.0, "p40": 8.0}


def latencies_path() -> Path:
    return Path(os.environ.get("ZORSE_LATENCIES", DATA_DIR / "model_latencies.json"))


def load_table(path=None) -> dict:
    p = Path(path) if path else latencies_path()
    if not p.exists():
        return {}
    with open(p) as f:
        return json.load(f)


def lookup(table: dict, model: str, gpu: str, seq: int, dtype: str, mbs: int) -> Optional[ModelLatencies]:
    try:
        e = table[model][gpu][str(seq)][dtype]
    except KeyError:
        return None
    if not isinstance(e, list):
        return None
    (fs, fi), (bs, bi) = e[0], e[1]
    fwd, bwd = fs * mbs + fi, bs * mbs + bi
    if len(e) >= 4:
        if len(e[2]) >= mbs:
            fwd = e[2][mbs - 1]
        if len(e[3]) >= mbs:
            bwd = e[3][mbs - 1]
    return ModelLatencies(float(fwd), float(bwd))


def analytic(model: str, gpu: str, seq: int, mbs: int, **overrides) -> ModelLatencies:
    spec = registry.get_spec(model, **overrides)
    blk = registry.make_block(spec)
    flops = blk.flops_per_token(seq) * mbs * seq
    tf = ANALYTIC_TFLOPS.get(gpu, 100.0)
    fwd = flops / (tf * 1e12) * 1e3
    return ModelLatencies(fwd, 2.0 * fwd)


def load_model_compute_latencies_per_gpu(model: str, gpus: list[str], seq: int, dtype: str, mbs: int,
                                         table: Optional[dict] = None) -> dict[str, ModelLatencies]:
    table = load_table() if table is None else table
    out = {}
    for g in sorted(set(gpus)):
        out[g] = lookup(table, model, g, seq, dtype, mbs) or analytic(model, g, seq, mbs)
    return out


def store(table: dict, model: str, gpu: str, seq: int, dtype: str, fwd_ms: list[float], bwd_ms: list[float]) -> None:
    """Adds a profile (times at microbatch sizes 1..n) with its least-squares line."""
    from ..utils.trace import fit_line

    fit = lambda ys: list(fit_line(ys))
    table.setdefault(model, {}).setdefault(gpu, {}).setdefault(str(seq), {})[dtype] = [fit(fwd_ms), fit(bwd_ms),
                                                                                      list(fwd_ms), list(bwd_ms)]


def head_and_embedding_ms(model: str, gpu: str, seq: int, mbs: int, vocab: int, **overrides) -> tuple[tuple, tuple]:
    """Analytic (forward, backward) times per microbatch of the output head and of the embedding:
    the head is two GEMM-sized passes (dgrad + wgrad) over [tokens, hidden] x [vocab, hidden] plus
    a cross-entropy pass over the logits; the embedding is a gather / scatter of the activations."""
    spec = registry.get_spec(model, vocab=vocab, **overrides)
    tf = ANALYTIC_TFLOPS.get(gpu, 100.0) * 1e12
    hbm = {"b200": 6.5e12}.get(gpu, 1.5e12)
    T = mbs * seq
    gemm = 2.0 * T * spec.hidden * (vocab or spec.vocab) / tf * 1e3
    ce = 2.0 * T * (vocab or spec.vocab) * 2 / hbm * 1e3
    emb = 2.0 * T * spec.hidden * 2 / hbm * 1e3
    return (gemm + 0.5 * ce, 2.0 * gemm + 0.5 * ce), (emb, 2.0 * emb)


def store_activation_bytes(table: dict, model: str, gpu: str, seq: int, dtype: str, act_bytes: list) -> None:
    """Peak bytes one block allocates while running forward + backward at microbatch sizes 1..n (measured by
    the layer profiler), kept beside the latencies under the `_activation_bytes` key."""
    table.setdefault("_activation_bytes", {}).setdefault(model, {}).setdefault(gpu, {}).setdefault(str(seq), {})[dtype] = \
        [int(x) for x in act_bytes]


def activation_bytes(table: dict, model: str, gpu: str, seq: int, dtype: str, mbs: int) -> Optional[float]:
    """Measured activation bytes of one block at microbatch size `mbs`: the measured value when the profile
    reaches that size, otherwise the value at the largest profiled size plus the median increase per extra
    sequence (reference utils/runtime_estimator.py:115-160 extrapolates with the same median increase)."""
    try:
        a = table["_activation_bytes"][model][gpu][str(seq)][dtype]
    except (KeyError, TypeError):
        return None
    if not a:
        return None
    if mbs <= len(a):
        return float(a[mbs - 1])
    inc = sorted(y - x for x, y in zip(a, a[1:]))
    step = inc[len(inc) // 2] if inc else float(a[0])
    return float(a[-1] + step * (mbs - len(a)))
