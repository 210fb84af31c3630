"""Builds libkfb200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python kernel-forge_b200/build.py [--force] [--verbose]

Each csrc/*.cu is compiled to build/<name>.o (in parallel, skipped when up to date) and the
objects are linked into kernelforge/libkfb200.so.  ptxas resource usage (registers, spills,
shared memory) of every kernel is kept in build/<name>.ptxas.txt.  No torch headers are used.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent
CSRC = PKG_ROOT / "csrc"
BUILD = PKG_ROOT / "build"
LIB = PKG_ROOT / "kernelforge" / "libkfb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
]


# per-source extra flags
EXTRA_FLAGS: dict[str, list[str]] = {}


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the kfb200 library needs the CUDA 12.8+ toolkit")
    return exe


def _deps_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG_ROOT.parent / "include" / "kfb200.h", Path(__file__)]
    return max(p.stat().st_mtime for p in hdrs if p.exists())


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    obj = BUILD / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, _deps_mtime()):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *EXTRA_FLAGS.get(src.name, []), "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (BUILD / (src.stem + ".ptxas.txt")).write_text(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), sources))
    if force or not LIB.exists() or LIB.stat().st_mtime < max(o.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
