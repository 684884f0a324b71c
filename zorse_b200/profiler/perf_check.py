"""Performance regression check: compares a `kernel_bench --out` file with the recorded B200
times in data/kernel_baseline_b200.json.

    python -m zorse_b200.profiler.kernel_bench --out new.json
    python -m zorse_b200.profiler.perf_check new.json [--baseline FILE] [--tolerance 0.10] [--update]

Exit status 1 if any kernel is slower than its recorded time by more than the tolerance;
`--update` rewrites the baseline with the new times (after an intended change).  Rows that the
baseline does not know (new kernels, candidates) are listed and ignored.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

DEFAULT = Path(__file__).resolve().parents[2] / "data" / "kernel_baseline_b200.json"


def key_of(row: dict) -> str:
    return f"{row['op']} | {row['shape']}"


def compare(rows: list[dict], baseline: dict, tolerance: float) -> dict:
    """{'slower': [(key, new_ms, old_ms)], 'faster': [...], 'same': n, 'unknown': [keys]}."""
    out = {"slower": [], "faster": [], "same": 0, "unknown": []}
    known = baseline["kernels"]
    for r in rows:
        k = key_of(r)
        if k not in known:
            out["unknown"].append(k)
            continue
        old, new = known[k]["ours_ms"], r["ours_ms"]
        if new > old * (1.0 + tolerance):
            out["slower"].append((k, new, old))
        elif new < old * (1.0 - tolerance):
            out["faster"].append((k, new, old))
        else:
            out["same"] += 1
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("results")
    ap.add_argument("--baseline", default=str(DEFAULT))
    ap.add_argument("--tolerance", type=float, default=None)
    ap.add_argument("--update", action="store_true")
    a = ap.parse_args(argv)
    rows = json.loads(Path(a.results).read_text())["rows"]
    baseline = json.loads(Path(a.baseline).read_text())
    tol = baseline.get("tolerance", 0.10) if a.tolerance is None else a.tolerance
    res = compare(rows, baseline, tol)
    for k, new, old in res["slower"]:
        print(f"SLOWER  {k}: {new:.4f} ms vs {old:.4f} ms recorded ({100 * (new / old - 1):+.0f} %)")
    for k, new, old in res["faster"]:
        print(f"faster  {k}: {new:.4f} ms vs {old:.4f} ms recorded ({100 * (new / old - 1):+.0f} %)")
    print(f"{res['same']} within {100 * tol:.0f} %, {len(res['faster'])} faster, {len(res['slower'])} slower, "
          f"{len(res['unknown'])} not in the baseline")
    if a.update:
        for r in rows:
            baseline["kernels"][key_of(r)] = {"ours_ms": round(r["ours_ms"], 4),
                                             **({"lib_ms": round(r["lib_ms"], 4)} if r.get("lib_ms") else {})}
        Path(a.baseline).write_text(json.dumps(baseline, indent=1))
        print(f"baseline updated: {a.baseline}")
    return 1 if res["slower"] else 0


if __name__ == "__main__":
    sys.exit(main())
