"""Phase timeline of the attention kernels that carry an in-kernel event trace (forward version 4,
backward version 2).

    python -m zorse_b200.profiler.attn_trace [--kernel fwd4|bwd2] [--S 4096 --heads 32 --kv_heads 32 --D 128]
                                             [--ctas 8] [--flags 0] [--cta 0] [--out FILE.json]

The kernel's first `--ctas` CTAs record (clock64, code) pairs per warp at phase boundaries.  For
one CTA this tool prints, per role, the mean / max number of SM clocks between consecutive
boundaries, i.e. where a key tile's time goes:

    softmax warp:  S ready -> row in registers -> maximum (and O rescale) -> first P half stored
                   -> second P half stored -> (waiting for the next S)
    MMA issuer:    what it waited for (V tile, P halves, K tile) and when it issued
    TMA producer:  slot free -> loads issued
(backward: S^T ready -> P^T stored -> dP^T ready -> dS^T stored -> dQ ready -> dQ drained.)

Decoding and the summary are plain Python (`decode`, `phase_stats`) and are unit-tested on CPU.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict

CODES = {1: "s_ready", 2: "s_loaded", 3: "max_done", 4: "p_half0", 5: "p_half1", 6: "epi_begin", 7: "epi_end",
         16: "mma_v_ready", 17: "mma_p0_ready", 18: "mma_p1_ready", 19: "mma_pv_issued", 20: "mma_k_ready",
         21: "mma_qk_issued", 32: "tma_slot_free", 33: "tma_issued"}


BWD_CODES = {1: "s_ready", 2: "p_done", 3: "dp_ready", 4: "ds_done", 5: "dq_ready", 6: "dq_drained",
             16: "mma_qdo_ready", 17: "mma_pds_ready", 18: "mma_def_issued", 19: "mma_a_issued", 20: "mma_dq_empty",
             21: "mma_b_issued", 32: "tma_stage_free", 33: "tma_issued"}


def decode(words, codes=None) -> list[tuple[int, str]]:
    """One warp's event words -> [(clock, name)], unused (zero) slots dropped."""
    codes = CODES if codes is None else codes
    out = []
    for w in words:
        w = int(w)
        if w == 0:
            continue
        out.append(((w >> 8) & ((1 << 55) - 1), codes.get(w & 0xFF, f"code{w & 0xFF}")))
    return out


def phase_stats(events: list[tuple[int, str]]) -> dict[str, dict]:
    """Durations between consecutive events of one warp, grouped by 'from->to'."""
    acc: dict[str, list[int]] = defaultdict(list)
    for (t0, a), (t1, b) in zip(events, events[1:]):
        acc[f"{a}->{b}"].append(t1 - t0)
    return {k: {"n": len(v), "mean": sum(v) / len(v), "max": max(v), "min": min(v), "total": sum(v)}
            for k, v in acc.items()}


def summarize(trace, cta: int, codes=None) -> dict:
    """trace: [ctas, warps, events] integer array-like (host). Returns {warp: {span, phases}}."""
    res = {}
    for w in range(len(trace[cta])):
        ev = decode(trace[cta][w], codes)
        if not ev:
            continue
        res[w] = {"events": len(ev), "span": ev[-1][0] - ev[0][0], "first": ev[0][0], "phases": phase_stats(ev)}
    return res


def format_summary(summary: dict) -> str:
    if not summary:
        return ("no events recorded for this CTA: the kernel returned before its first trace point "
                "(check the status word), or the CTA index is beyond the traced ones")
    lines = []
    t0 = min(v["first"] for v in summary.values()) if summary else 0
    for w, v in sorted(summary.items()):
        lines.append(f"warp {w}: {v['events']} events over {v['span']} clocks (starts at +{v['first'] - t0})")
        for k, st in sorted(v["phases"].items(), key=lambda kv: -kv[1]["total"]):
            lines.append(f"    {k:32s} n={st['n']:4d} mean={st['mean']:9.1f} min={st['min']:7d} max={st['max']:7d} "
                         f"total={st['total']}")
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="fwd4", choices=["fwd4", "bwd2", "bwd3"],
                    help="bwd3: the dK / dV kernel of the two-kernel backward (same phase codes as bwd2, no dQ phases)")
    ap.add_argument("--S", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv_heads", type=int, default=32)
    ap.add_argument("--D", type=int, default=128)
    ap.add_argument("--window", type=int, default=0)
    ap.add_argument("--ctas", type=int, default=8)
    ap.add_argument("--cta", type=int, default=0, help="which traced CTA to print (0 = heaviest query pair of head 0)")
    ap.add_argument("--flags", type=int, default=0)
    ap.add_argument("--out", default=None)
    ap.add_argument("--device", default="cuda", help=argparse.SUPPRESS)     # "cpu" only for the tool's own dry-run test
    a = ap.parse_args(argv)
    import torch

    from zorse_b200.ops import sm100 as k

    dev = a.device
    g = torch.Generator(device=dev).manual_seed(0)
    qkv = (torch.randn(a.S, (a.heads + 2 * a.kv_heads) * a.D, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    codes = CODES
    if a.kernel == "fwd4":
        for _ in range(2):
            k.flash_fwd(qkv, 1, a.S, a.heads, a.kv_heads, a.D, True, a.window, version=4, flags=a.flags)
        buf = k.flash_fwd4_trace_buffer(dev, a.ctas)
        k.flash_fwd(qkv, 1, a.S, a.heads, a.kv_heads, a.D, True, a.window, version=4, flags=a.flags, trace=buf,
                    trace_ctas=a.ctas)
    else:
        codes = BWD_CODES
        do = (torch.randn(a.S, a.heads * a.D, device=dev, generator=g) * 0.5).to(torch.bfloat16)
        out, lse = k.flash_fwd(qkv, 1, a.S, a.heads, a.kv_heads, a.D, True, a.window)
        ver = 3 if a.kernel == "bwd3" else 2
        for _ in range(2):
            k.flash_bwd(do, qkv, out, lse, 1, a.S, a.heads, a.kv_heads, a.D, True, a.window, version=ver)
        buf = k.flash_bwd2_trace_buffer(dev, a.ctas)
        k.flash_bwd(do, qkv, out, lse, 1, a.S, a.heads, a.kv_heads, a.D, True, a.window, version=ver, trace=buf,
                    trace_ctas=a.ctas)
    if dev == "cuda":
        torch.cuda.synchronize()
    k.check_status()
    host = buf.cpu().tolist()
    summ = summarize(host, a.cta, codes)
    print(format_summary(summ))
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"args": vars(a), "cta": a.cta, "summary": summ,
                       "events": {w: decode(host[a.cta][w], codes) for w in range(len(host[a.cta]))}}, f)


if __name__ == "__main__":
    main()
