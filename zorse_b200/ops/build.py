"""Builds the sm_100a kernel library in-tree with nvcc (no torch headers involved).

Every `.cu` file under `csrc/` is compiled to an object with
`-gencode arch=compute_100a,code=sm_100a` and linked into
`zorse_b200/_C/libzorse_sm100.so`, a plain C-ABI shared library that
`zorse_b200.ops.sm100` loads with ctypes.  Objects are rebuilt only when their source
(or any header under `csrc/`) is newer.

    python -m zorse_b200.ops.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

REPO = Path(__file__).resolve().parents[2]
CSRC = REPO / "csrc"
OUT_DIR = REPO / "zorse_b200" / "_C"
OBJ_DIR = OUT_DIR / "obj"
LIB = OUT_DIR / "libzorse_sm100.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the sm_100a kernels cannot be built")
    return nvcc


def sources() -> list[Path]:
    return sorted(CSRC.rglob("*.cu"))


def _newest_header_mtime() -> float:
    hs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool, extra=()) -> str:
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr)
    # compile times change from run to run; leaving them out keeps the tracked summary stable
    kept = "\n".join(ln for ln in r.stderr.splitlines() if "Compile time" not in ln)
    obj.with_suffix(".log").write_text(f"==== {src.relative_to(CSRC)}\n{kept}\n")
    return r.stderr


DEBUG_LIB = OUT_DIR / "libzorse_sm100_dbg.so"


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    """`debug_bounds`: the checking build (`-DZB_DEBUG_BOUNDS=1`, own object directory and library name):
    kernels compare tile coordinates, shard offsets and flag indices with the extents they were given and
    report through the status word instead of touching memory outside them.  Loaded instead of the normal
    library when ZORSE_DEBUG_BOUNDS=1."""
    if debug_bounds:
        return _build(force, verbose, OUT_DIR / "obj_dbg", DEBUG_LIB, ["-DZB_DEBUG_BOUNDS=1"], write_log=False)
    return _build(force, verbose, OBJ_DIR, LIB, [], write_log=True)


def _build(force: bool, verbose: bool, OBJ_DIR: Path, LIB: Path, extra: list, write_log: bool) -> Path:
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime()
    jobs = []
    objs = []
    for src in sources():
        obj = OBJ_DIR / (str(src.relative_to(CSRC)).replace("/", "__")[:-3] + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = [ex.submit(_compile_one, nvcc, s, o, verbose, tuple(extra)) for s, o in jobs]
            for f in futs:
                f.result()
        # registers / spills / shared memory of every kernel, one section per source file
        if write_log:
            (OUT_DIR / "ptxas.log").write_text("\n".join(o.with_suffix(".log").read_text() for o in objs
                                                      if o.with_suffix(".log").exists()))
    if jobs or not LIB.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--debug-bounds", action="store_true", help="the checking build (libzorse_sm100_dbg.so)")
    a = ap.parse_args(argv)
    lib = build(force=a.force, verbose=a.verbose, debug_bounds=a.debug_bounds)
    print(lib)
    return 0


if __name__ == "__main__":
    sys.exit(main())
