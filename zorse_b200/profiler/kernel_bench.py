"""Times this repository's sm_100a kernels against the library kernels the reference
would reach (cuBLAS through torch.matmul, SDPA/flash attention, ATen fused ops), at the
shapes of the benchmark configurations.

    python -m zorse_b200.profiler.kernel_bench [--out FILE.json] [--only gemm,attn,...]

Timing: CUDA events on the launching stream, `--warmup` untimed runs, then `--iters` timed
runs with a write larger than L2 between runs so no operand is served from cache; the
figure reported is the median.  Roofline fractions use the peaks given with `--peaks FILE`
(or `--peak_hbm_gbs` / `--peak_bf16_tflops`), else B200 fallback figures.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]


def _peaks(path=None, hbm_gbs=None, bf16_tflops=None):
    """Roofline denominators: from `--peaks FILE` (JSON with `hbm_gbs` and `bf16_tflops`, e.g. a copy-bandwidth
    and library-GEMM measurement taken on the same machine), from the two flags, or B200 fallback figures."""
    if path:
        d = json.loads(Path(path).read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    if hbm_gbs and bf16_tflops:
        return {"hbm_gbs": float(hbm_gbs), "bf16_tflops": float(bf16_tflops), "source": "flags"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_flush = None
DEV = "cuda"            # "cpu" only in the tool's own dry-run test (stand-in library, small shapes)
FLUSH_BYTES = 256 * 1024 * 1024
GEMM_SHAPES = [
    # name, M(tokens), N, K
    ("7b qkv", 4096, 12288, 4096), ("7b o", 4096, 4096, 4096), ("7b gate_up", 4096, 22016, 4096),
    ("7b down", 4096, 4096, 11008), ("7b head", 4096, 32000, 4096),
    ("1b gate_up", 2048, 16384, 2048), ("square 8192", 8192, 8192, 8192),
]
ATTN_CASES = [("7b", 1, 4096, 32, 32, 128, 0), ("1b", 1, 2048, 32, 8, 64, 0), ("mistral", 1, 8192, 32, 8, 128, 4096)]
ELEMENTWISE_DIMS = (4096, 4096, 11008, 32000, 202_383_360 // 2)      # tokens, hidden, ffn, vocab, Adam elements


def time_fn(fn, warmup=3, iters=10):
    global _flush
    if _flush is None or _flush.device.type != DEV:
        _flush = torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=DEV)
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        _flush.zero_()
        if DEV == "cuda":
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        else:
            import time

            t0 = time.perf_counter()
            fn()
            ts.append(max((time.perf_counter() - t0) * 1e3, 1e-6))
    return statistics.median(ts)


def bench_gemm(k, peaks, rows):
    for name, M, N, K in GEMM_SHAPES:
        a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
        dy = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
        out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
        dx = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
        gw = torch.zeros(N, K, device=DEV, dtype=torch.float32)
        fl = 2.0 * M * N * K
        gw = torch.zeros(N, K, device=DEV, dtype=torch.bfloat16)
        for kern in ("1cta", "2cta"):
            for kind, ours, lib in (
                ("fwd", lambda: k.gemm(a, w, out, kernel=kern), lambda: torch.matmul(a, w.t(), out=out)),
                ("dgrad", lambda: k.gemm(dy, w, dx, b_mn=True, kernel=kern), lambda: torch.matmul(dy, w, out=dx)),
                ("wgrad+=", lambda: k.gemm(dy, a, gw, a_mn=True, b_mn=True, accumulate=True, kernel=kern),
                 lambda: torch.matmul(dy.t(), a)),
            ):
                t_o, t_l = time_fn(ours), time_fn(lib)
                rows.append({"op": f"gemm {kind} {kern}", "shape": f"{name} M{M} N{N} K{K}", "ours_ms": t_o, "lib_ms": t_l,
                             "ours_tflops": fl / t_o / 1e9, "lib_tflops": fl / t_l / 1e9,
                             "frac_of_peak": fl / t_o / 1e9 / peaks["bf16_tflops"]})
        if os.environ.get("ZORSE_BENCH_CANDIDATES") == "1":     # kernels not yet validated on hardware
            t_o = time_fn(lambda: k.gemm(dy, a, gw, a_mn=True, b_mn=True, accumulate=True, kernel="2cta_accpf"))
            rows.append({"op": "gemm wgrad+= 2cta_accpf", "shape": f"{name} M{M} N{N} K{K}", "ours_ms": t_o, "lib_ms": None,
                         "ours_tflops": fl / t_o / 1e9, "lib_tflops": None,
                         "frac_of_peak": fl / t_o / 1e9 / peaks["bf16_tflops"]})
        k.check_status()
        del a, w, dy, out, dx, gw


def bench_attn(k, peaks, rows):
    import torch.nn.functional as F

    for name, B, S, Hq, Hkv, D, win in ATTN_CASES:
        qkv = torch.randn(B * S, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16)
        do = torch.randn(B * S, Hq * D, device=DEV, dtype=torch.bfloat16)
        out, lse = k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, win)
        x = qkv.view(B, S, Hq + 2 * Hkv, D)
        q = x[:, :, :Hq].transpose(1, 2)
        kk = x[:, :, Hq:Hq + Hkv].transpose(1, 2)
        v = x[:, :, Hq + Hkv:].transpose(1, 2)
        if win:
            pairs = sum(min(i + 1, win) for i in range(S))
        else:
            pairs = S * (S + 1) // 2
        fl_f = 4.0 * pairs * D * Hq * B
        t_o = time_fn(lambda: k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, win))
        cand = os.environ.get("ZORSE_BENCH_CANDIDATES") == "1"   # kernels not yet validated on hardware
        for ver, fl in [(1, 0), (2, 0)] + ([(4, 0), (4, 1), (4, 2)] if cand else []):
            t_v = time_fn(lambda: k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, win, version=ver, flags=fl))
            rows.append({"op": f"flash fwd v{ver}" + (f" mode{fl}" if fl else ""), "shape": f"{name} S{S} Hq{Hq} Hkv{Hkv} D{D} win{win}", "ours_ms": t_v,
                         "lib_ms": None, "ours_tflops": fl_f / t_v / 1e9, "frac_of_peak": fl_f / t_v / 1e9 / peaks["bf16_tflops"]})
        t_l = None
        if not win:
            try:
                t_l = time_fn(lambda: F.scaled_dot_product_attention(q, kk, v, is_causal=True, enable_gqa=True))
            except Exception:
                t_l = None
        rows.append({"op": "flash fwd", "shape": f"{name} S{S} Hq{Hq} Hkv{Hkv} D{D} win{win}", "ours_ms": t_o,
                     "lib_ms": t_l, "ours_tflops": fl_f / t_o / 1e9,
                     "lib_tflops": None if t_l is None else fl_f / t_l / 1e9,
                     "frac_of_peak": fl_f / t_o / 1e9 / peaks["bf16_tflops"]})
        if hasattr(k, "flash_bwd"):
            t_b = time_fn(lambda: k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D, True, win))
            t_lb = None
            if not win:
                try:
                    qg, kg, vg = (t.detach().clone().requires_grad_(True) for t in (q, kk, v))
                    og = F.scaled_dot_product_attention(qg, kg, vg, is_causal=True, enable_gqa=True)
                    dog = do.view(B, S, Hq, D).transpose(1, 2)
                    t_lb = time_fn(lambda: torch.autograd.grad(og, (qg, kg, vg), dog, retain_graph=True))
                except Exception:
                    t_lb = None
            if cand:
                t_b2 = time_fn(lambda: k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D, True, win, version=2))
                rows.append({"op": "flash bwd v2", "shape": f"{name} S{S} Hq{Hq} Hkv{Hkv} D{D} win{win}", "ours_ms": t_b2,
                             "lib_ms": None, "ours_tflops": 2.5 * fl_f / t_b2 / 1e9,
                             "frac_of_peak": 2.5 * fl_f / t_b2 / 1e9 / peaks["bf16_tflops"]})
            rows.append({"op": "flash bwd", "shape": f"{name} S{S} Hq{Hq} Hkv{Hkv} D{D} win{win}", "ours_ms": t_b,
                         "lib_ms": t_lb, "ours_tflops": 2.5 * fl_f / t_b / 1e9,
                         "lib_tflops": None if t_lb is None else 2.5 * fl_f / t_lb / 1e9,
                         "frac_of_peak": 2.5 * fl_f / t_b / 1e9 / peaks["bf16_tflops"]})
        k.check_status()


def bench_elementwise(k, peaks, rows):
    import torch.nn.functional as F

    T, H, Fd, V, n_adam = ELEMENTWISE_DIMS
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(H, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    y, st = k.norm_fwd(x, w, None, 1e-5, False)
    gw = torch.zeros(H, device=DEV, dtype=torch.float32)

    def add(op, shape, t_o, t_l, nbytes):
        rows.append({"op": op, "shape": shape, "ours_ms": t_o, "lib_ms": t_l, "ours_gbs": nbytes / t_o / 1e6,
                     "frac_of_peak": nbytes / t_o / 1e6 / peaks["hbm_gbs"]})

    add("rmsnorm fwd", f"T{T} H{H}", time_fn(lambda: k.norm_fwd(x, w, None, 1e-5, False)),
        time_fn(lambda: F.rms_norm(x, (H,), w, 1e-5)), 2 * T * H * 2)
    add("rmsnorm bwd", f"T{T} H{H}", time_fn(lambda: k.norm_bwd(dy, x, w, st, None, gw, None, False, version=1)), None,
        3 * T * H * 2)
    if os.environ.get("ZORSE_BENCH_CANDIDATES") == "1":
        add("rmsnorm fwd v2", f"T{T} H{H}", time_fn(lambda: k.norm_fwd(x, w, None, 1e-5, False, version=2)), None,
            2 * T * H * 2)
        add("rmsnorm bwd v2", f"T{T} H{H}", time_fn(lambda: k.norm_bwd(dy, x, w, st, None, gw, None, False, version=2)),
            None, 3 * T * H * 2)
    gu = torch.randn(T, 2 * Fd, device=DEV, dtype=torch.bfloat16)
    dout = torch.randn(T, Fd, device=DEV, dtype=torch.bfloat16)
    add("swiglu fwd", f"T{T} F{Fd}", time_fn(lambda: k.swiglu_fwd(gu)),
        time_fn(lambda: F.silu(gu[:, :Fd]) * gu[:, Fd:]), 3 * T * Fd * 2)
    add("swiglu bwd", f"T{T} F{Fd}", time_fn(lambda: k.swiglu_bwd(gu, dout)), None, 5 * T * Fd * 2)
    logits = torch.randn(T, V, device=DEV, dtype=torch.bfloat16)
    tg = torch.randint(0, V, (T,), device=DEV)
    add("cross-entropy fwd+bwd", f"T{T} V{V}", time_fn(lambda: k.cross_entropy(logits, tg, 1.0, dlogits=logits)),
        None, 2 * T * V * 2)
    n = n_adam
    p, m, v = (torch.zeros(n, device=DEV) for _ in range(3))
    g = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    p16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    add("adam (bf16 grad)", f"n{n}", time_fn(lambda: k.adam_step(p, m, v, g, p16, lr=1e-3, beta1=0.9, beta2=0.999,
                                                                   eps=1e-8, weight_decay=0.0, step=1)),
        None, n * (12 + 2 + 12 + 2))
    qkv = torch.randn(T, 3 * H, device=DEV, dtype=torch.bfloat16)
    from zorse_b200.ops import ref
    cs = ref.rope_table(T, 128, 1e4, DEV)
    add("rope (q,k in place)", f"T{T} 64 heads d128", time_fn(lambda: k.rope_(qkv, cs, T, 64, 128)), None,
        2 * T * 2 * H * 2)
    k.check_status()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--only", default="gemm,attn,elementwise")
    ap.add_argument("--peaks", default=None, help="JSON file with measured hbm_gbs and bf16_tflops of this machine")
    ap.add_argument("--peak_hbm_gbs", type=float, default=None)
    ap.add_argument("--peak_bf16_tflops", type=float, default=None)
    a = ap.parse_args(argv)
    from zorse_b200.ops import sm100 as k

    k.lib()
    peaks = _peaks(a.peaks, a.peak_hbm_gbs, a.peak_bf16_tflops)
    rows: list[dict] = []
    only = a.only.split(",")
    if "gemm" in only:
        bench_gemm(k, peaks, rows)
    if "attn" in only:
        bench_attn(k, peaks, rows)
    if "elementwise" in only:
        bench_elementwise(k, peaks, rows)
    for r in rows:
        lib = "" if r.get("lib_ms") is None else f" lib {r['lib_ms']:.3f} ms"
        perf = f"{r['ours_tflops']:.0f} TFLOP/s" if "ours_tflops" in r else f"{r['ours_gbs']:.0f} GB/s"
        print(f"{r['op']:24s} {r['shape']:40s} ours {r['ours_ms']:.3f} ms{lib}  {perf}  "
              f"{100 * r['frac_of_peak']:.0f}% of {peaks['source']} peak")
    if a.out:
        Path(a.out).write_text(json.dumps({"peaks": peaks, "rows": rows}, indent=1))


if __name__ == "__main__":
    main()
