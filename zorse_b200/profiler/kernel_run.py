"""Runs ONE of this repository's kernels a few times on a small, larger-than-L2 case, for
`ncu` captures (`ncu --set full --clock-control none -k regex:<name> -c 2 python -m
zorse_b200.profiler.kernel_run <case>`).  Holds well under a few GB on the device.

cases: gemm_fwd | gemm_dgrad | gemm_wgrad | flash_fwd1 | flash_fwd2 | flash_fwd4 | flash_fwd4p | flash_fwd4q | flash_bwd | flash_bwd2 |
       flash_bwd3 | flash_bwd3_dkv | flash_bwd3_dq | rmsnorm | rmsnorm_bwd | layernorm_bwd | rope | swiglu_fwd | swiglu_bwd |
       embedding_fwd | embedding_bwd | adam | ce
Prints the median CUDA-event time of the repetitions (a 256 MB write between them keeps operands out of L2).
"""
from __future__ import annotations

import sys

import torch


def main(argv=None):
    case = (argv or sys.argv[1:])[0]
    reps = int((argv or sys.argv[1:])[1]) if len(argv or sys.argv[1:]) > 1 else 3
    from zorse_b200.ops import sm100 as k

    k.lib()
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: (torch.randn(*s, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    if case.startswith("gemm"):
        M, N, K = 4096, 11008, 4096          # 34 + 90 + 90 MB
        a, w, dy = rnd(M, K), rnd(N, K), rnd(M, N)
        out, dx = torch.empty(M, N, device=dev, dtype=torch.bfloat16), torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        gw = torch.zeros(N, K, device=dev, dtype=torch.bfloat16)
        fn = {"gemm_fwd": lambda: k.gemm(a, w, out), "gemm_dgrad": lambda: k.gemm(dy, w, dx, b_mn=True),
              "gemm_wgrad": lambda: k.gemm(dy, a, gw, a_mn=True, b_mn=True, accumulate=True)}[case]
    elif case.startswith("flash"):
        B, S, Hq, Hkv, D = 1, 4096, 32, 32, 128   # qkv 100 MB
        qkv, do = rnd(B * S, (Hq + 2 * Hkv) * D), rnd(B * S, Hq * D)
        out, lse = k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 0)
        fn = {"flash_fwd1": lambda: k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 0, version=1),
              "flash_fwd2": lambda: k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 0, version=2),
              "flash_fwd4": lambda: k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 0, version=4, flags=0),
              "flash_fwd4p": lambda: k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 0, version=4, flags=1),
              "flash_fwd4q": lambda: k.flash_fwd(qkv, B, S, Hq, Hkv, D, True, 0, version=4, flags=2),
              "flash_bwd": lambda: k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D, True, 0, version=1),
              "flash_bwd2": lambda: k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D, True, 0, version=2),
              "flash_bwd3": lambda: k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D, True, 0, version=3),
              "flash_bwd3_dkv": lambda: k._flash_bwd3(do, qkv, out, lse, B, S, Hq, Hkv, D, True, 0, None, parts=1),
              "flash_bwd3_dq": lambda: k._flash_bwd3(do, qkv, out, lse, B, S, Hq, Hkv, D, True, 0, None, parts=2)}[case]
        if case == "flash_bwd3_dq":
            k.flash_bwd(do, qkv, out, lse, B, S, Hq, Hkv, D, True, 0, version=3)   # fills the statistics
    elif case == "rmsnorm":
        x, w = rnd(32768, 4096), torch.ones(4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: k.norm_fwd(x, w, None, 1e-5, False)
    elif case in ("rmsnorm_bwd", "layernorm_bwd"):
        ln = case.startswith("layer")
        x, w, dy, dres = rnd(32768, 4096), torch.ones(4096, device=dev, dtype=torch.bfloat16), rnd(32768, 4096), rnd(32768, 4096)
        b = torch.zeros(4096, device=dev, dtype=torch.bfloat16) if ln else None
        _, st = k.norm_fwd(x, w, b, 1e-5, ln)
        dw = torch.zeros(4096, device=dev)
        db = torch.zeros(4096, device=dev) if ln else None
        fn = lambda: k.norm_bwd(dy, x, w, st, dres, dw, db, ln)
    elif case == "rope":
        S, H, D = 4096, 64, 128                                  # q and k heads of a 7B block, 8 sequences: 537 MB
        buf = rnd(8 * S, 3 * 32 * D)
        pos = torch.arange(S, device=dev, dtype=torch.float32)[:, None]
        inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D))[None, :]
        cs = torch.cat([torch.cos(pos * inv), torch.sin(pos * inv)], dim=1).contiguous()
        fn = lambda: k.rope_(buf, cs, S, H, D)
    elif case in ("swiglu_fwd", "swiglu_bwd"):
        gu, dh = rnd(16384, 2 * 11008), rnd(16384, 11008)        # 721 MB + 361 MB
        fn = (lambda: k.swiglu_fwd(gu)) if case.endswith("fwd") else (lambda: k.swiglu_bwd(gu, dh))
    elif case in ("embedding_fwd", "embedding_bwd"):
        ids = torch.randint(0, 32000, (65536,), device=dev)
        table, dout = rnd(32000, 4096), rnd(65536, 4096)
        dtable = torch.zeros(32000, 4096, device=dev)
        fn = (lambda: k.embedding_fwd(ids, table)) if case.endswith("fwd") else (lambda: k.embedding_bwd(ids, dout, dtable))
    elif case == "adam":
        n = 64 * 1024 * 1024
        p, m, v = (torch.zeros(n, device=dev) for _ in range(3))
        gr, p16 = rnd(n), torch.empty(n, device=dev, dtype=torch.bfloat16)
        fn = lambda: k.adam_step(p, m, v, gr, p16, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=1)
    elif case == "ce":
        lg, tg = rnd(4096, 32000), torch.randint(0, 32000, (4096,), device=dev)
        fn = lambda: k.cross_entropy(lg, tg, 1.0, dlogits=lg)
    else:
        raise SystemExit(__doc__)
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    ts = []
    for _ in range(reps):
        flush.add_(1.0)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        fn()
        ev1.record()
        torch.cuda.synchronize()
        ts.append(ev0.elapsed_time(ev1))
    k.check_status()
    print("ok", case, f"median {sorted(ts)[len(ts) // 2]:.4f} ms over {reps} runs")


if __name__ == "__main__":
    main()
