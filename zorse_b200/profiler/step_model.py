"""Where a training step's time goes, from the recorded kernel timings.

    python -m zorse_b200.profiler.step_model [--measured_ms 12450] [--timings data/kernel_baseline_b200.json]

Adds up, for the headline configuration (Llama-2-7B, sequence 4096, microbatch 1, 64 microbatches
on one GPU), how often each kernel of a transformer block runs per step times its recorded
isolated time (CUDA events, cold L2, burst clocks), per group of kernels, next to what the library
kernels the reference would reach take for the same work.  With `--measured_ms` (the step time the
benchmark reported) the last line gives the part of the step the isolated timings do not explain:
sustained clocks under the power cap are lower than burst clocks, plus launch gaps, the optimizer
and host copies.  The table says which kernels are worth work: a group's share of the step is the
most a faster kernel for it can win.
"""
from __future__ import annotations

import argparse
import json
import os

# (group, key in the timings file, launches per block and microbatch)
BLOCK_7B = [
    ("gemm fwd", "gemm fwd 2cta | 7b qkv M4096 N12288 K4096", 1),
    ("gemm fwd", "gemm fwd 2cta | 7b o M4096 N4096 K4096", 1),
    ("gemm fwd", "gemm fwd 2cta | 7b gate_up M4096 N22016 K4096", 1),
    ("gemm fwd", "gemm fwd 2cta | 7b down M4096 N4096 K11008", 1),
    ("gemm dgrad", "gemm dgrad 2cta | 7b qkv M4096 N12288 K4096", 1),
    ("gemm dgrad", "gemm dgrad 2cta | 7b o M4096 N4096 K4096", 1),
    ("gemm dgrad", "gemm dgrad 2cta | 7b gate_up M4096 N22016 K4096", 1),
    ("gemm dgrad", "gemm dgrad 2cta | 7b down M4096 N4096 K11008", 1),
    ("gemm wgrad", "gemm wgrad+= 2cta | 7b qkv M4096 N12288 K4096", 1),
    ("gemm wgrad", "gemm wgrad+= 2cta | 7b o M4096 N4096 K4096", 1),
    ("gemm wgrad", "gemm wgrad+= 2cta | 7b gate_up M4096 N22016 K4096", 1),
    ("gemm wgrad", "gemm wgrad+= 2cta | 7b down M4096 N4096 K11008", 1),
    ("attention fwd", "flash fwd | 7b S4096 Hq32 Hkv32 D128 win0", 1),
    ("attention bwd", "flash bwd | 7b S4096 Hq32 Hkv32 D128 win0", 1),
    ("norm", "rmsnorm fwd | T4096 H4096", 2),
    ("norm", "rmsnorm bwd | T4096 H4096", 2),
    ("elementwise", "swiglu fwd | T4096 F11008", 1),
    ("elementwise", "swiglu bwd | T4096 F11008", 1),
    ("elementwise", "rope (q,k in place) | T4096 64 heads d128", 2),
]
# once per microbatch (output layer) and once per block and step (optimizer on a block's parameters)
HEAD_7B = [
    ("head", "gemm fwd 2cta | 7b head M4096 N32000 K4096", 1),
    ("head", "gemm dgrad 2cta | 7b head M4096 N32000 K4096", 1),
    ("head", "gemm wgrad+= 2cta | 7b head M4096 N32000 K4096", 1),
    ("head", "cross-entropy fwd+bwd | T4096 V32000", 1),
    ("head", "rmsnorm fwd | T4096 H4096", 1),
    ("head", "rmsnorm bwd | T4096 H4096", 1),
]
ADAM_PER_BLOCK = ("optimizer", "adam (bf16 grad) | n101191680", 2)   # 202 M parameters per block


def step_model(timings: dict, layers: int = 32, microbatches: int = 64) -> dict:
    """{group: {"ours_ms", "lib_ms" (None where no library time was recorded)}} per step."""
    out: dict = {}

    def add(group, key, count):
        e = timings[key]
        g = out.setdefault(group, {"ours_ms": 0.0, "lib_ms": 0.0, "lib_complete": True})
        g["ours_ms"] += count * e["ours_ms"]
        if "lib_ms" in e:
            g["lib_ms"] += count * e["lib_ms"]
        else:
            g["lib_ms"] += count * e["ours_ms"]      # no library figure: count our own time on both sides
            g["lib_complete"] = False

    for group, key, n in BLOCK_7B:
        add(group, key, n * layers * microbatches)
    for group, key, n in HEAD_7B:
        add(group, key, n * microbatches)
    add(ADAM_PER_BLOCK[0], ADAM_PER_BLOCK[1], ADAM_PER_BLOCK[2] * layers)
    return out


def format_table(model: dict, measured_ms=None) -> str:
    total = sum(g["ours_ms"] for g in model.values())
    total_lib = sum(g["lib_ms"] for g in model.values())
    rows = ["| kernels | per step, ours (ms) | share of the sum | library kernels (ms) | ours / library |", "|---|---|---|---|---|"]
    for name, g in sorted(model.items(), key=lambda kv: -kv[1]["ours_ms"]):
        mark = "" if g["lib_complete"] else " (partly our own time: no library figure)"
        rows.append(f"| {name} | {g['ours_ms']:.0f} | {g['ours_ms'] / total:.1%} | {g['lib_ms']:.0f}{mark} | "
                    f"{g['ours_ms'] / g['lib_ms']:.2f} |")
    rows.append(f"| sum of isolated kernel times | {total:.0f} | 100% | {total_lib:.0f} | {total / total_lib:.2f} |")
    if measured_ms:
        rows.append(f"| measured step | {measured_ms:.0f} | | | |")
        rows.append(f"| not explained by isolated timings | {measured_ms - total:.0f} ({(measured_ms - total) / measured_ms:.1%} of the step) | | | |")
    return "\n".join(rows)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ap.add_argument("--timings", default=os.path.join(here, "data", "kernel_baseline_b200.json"))
    ap.add_argument("--measured_ms", type=float, default=None)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--microbatches", type=int, default=64)
    a = ap.parse_args(argv)
    with open(a.timings) as f:
        t = json.load(f)
    print(format_table(step_model(t.get("kernels", t), a.layers, a.microbatches), a.measured_ms))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
