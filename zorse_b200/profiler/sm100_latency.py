"""Latencies and issue costs of the sm_100a building blocks, measured inside one CTA with
clock64 (csrc/bench/latency_probe.cu):

    python -m zorse_b200.profiler.sm100_latency [--runs 5] [--out FILE.json]

Prints, in SM clocks (median over runs): TMEM load / store round trips, mbarrier hand-off
between warps, tcgen05.mma issue -> commit -> barrier observed for 1 / 8 / 16 / 32 MMAs of
128 x 128 x 16 (and the marginal clocks per MMA), and the cost of 1024 ex2 / fma / polynomial
exp2 per lane with one and two warps per scheduler.  These are the constants behind the
per-tile budgets quoted in the attention kernels' headers.
"""
from __future__ import annotations

import argparse
import json
import statistics

NAMES = {0: "tmem_ld_x32", 1: "tmem_ld_4x32", 2: "tmem_st_x32", 3: "mbarrier_handoff", 4: "mma_1", 5: "mma_8",
         6: "mma_16", 7: "mma_32", 8: "mma_8_observed_by_other_warp", 9: "ex2_1024_1warp_per_sched",
         10: "ex2_1024_2warps_per_sched", 11: "fma_1024_1warp_per_sched", 12: "fma_1024_2warps_per_sched",
         13: "exp2_poly_1024_1warp_per_sched"}


def derive(med: dict) -> dict:
    """Secondary figures from the medians (clocks)."""
    d = {}
    if med.get("mma_32") and med.get("mma_8"):
        d["clocks_per_mma_128x128x16"] = (med["mma_32"] - med["mma_8"]) / 24.0
        d["mma_fixed_latency"] = med["mma_8"] - 8 * d["clocks_per_mma_128x128x16"]
    for k in ("ex2_1024_1warp_per_sched", "ex2_1024_2warps_per_sched", "fma_1024_1warp_per_sched",
              "fma_1024_2warps_per_sched", "exp2_poly_1024_1warp_per_sched"):
        if med.get(k):
            d[k.replace("_1024", "_clocks_per_op")] = med[k] / 1024.0
    return d


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--runs", type=int, default=5)
    ap.add_argument("--out", default=None)
    ap.add_argument("--device", default="cuda", help=argparse.SUPPRESS)     # "cpu" only for the tool's own dry-run test
    a = ap.parse_args(argv)
    import ctypes

    import torch

    from zorse_b200.ops import sm100 as k

    lib = k.lib()
    n = lib.zb_latency_probe_count()
    runs = []
    for _ in range(a.runs):
        cuda = a.device == "cuda"
        out = torch.zeros(n, dtype=torch.int64, device=a.device)
        sink = torch.zeros(288, dtype=torch.float32, device=a.device)
        rc = lib.zb_latency_probe(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(sink.data_ptr()),
                                  ctypes.c_void_p(k.status_word(a.device).data_ptr()),
                                  ctypes.c_void_p(torch.cuda.current_stream().cuda_stream if cuda else 0))
        if rc != 0:
            raise RuntimeError(lib.zb_last_error().decode())
        if cuda:
            torch.cuda.synchronize()
        k.check_status()
        runs.append(out.cpu().tolist())
    med = {NAMES[i]: statistics.median(r[i] for r in runs) for i in NAMES}
    extra = derive(med)
    for name, v in med.items():
        print(f"{name:36s} {v:10.0f} clocks")
    for name, v in extra.items():
        print(f"{name:36s} {v:10.2f}")
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"median_clocks": med, "derived": extra, "runs": runs}, f, indent=1)


if __name__ == "__main__":
    main()
