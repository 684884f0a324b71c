#!/bin/bash
# Environment check + kernel build for zorse-b200 (the reference's setup.sh creates a conda env
# with pinned torch / transformers / flash-attn; this framework needs only PyTorch >= 2.6 with
# CUDA 12.8+, nvcc for sm_100a, and optionally networkx / scikit-learn for the planner).
set -e
python - <<'PY'
import importlib, sys
for m, need in [("torch", True), ("networkx", True), ("numpy", True), ("sklearn", False), ("pymetis", False), ("matplotlib", False)]:
    try:
        importlib.import_module(m); print(f"{m:12s} ok")
    except Exception:
        print(f"{m:12s} {'MISSING (required)' if need else 'missing (optional)'}")
        if need: sys.exit(1)
PY
python -m zorse_b200.ops.build
echo "built $(python -c 'from zorse_b200.ops import build; print(build.LIB)')"
