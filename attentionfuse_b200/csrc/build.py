"""Build the C-ABI shared library (libattnfuse_b200.so) for sm_100a, in-tree.

Every .cu in this directory is compiled to an object with nvcc and linked into one shared
library next to the sources.  The CUDA runtime is linked statically, so the library loads
(and its symbols can be inspected) on machines without a GPU or driver.

    python -m attentionfuse_b200.csrc.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
LIB = HERE / "libattnfuse_b200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-I", str(ROOT / "include"), "-I", str(HERE),
]


def _stamp(src: Path) -> str:
    h = hashlib.sha1()
    for f in [src, *sorted(HERE.glob("*.cuh")), ROOT / "include" / "attnfuse_b200.h"]:
        h.update(f.read_bytes())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    obj = src.with_suffix(".o")
    stamp_file = src.with_suffix(".o.stamp")
    stamp = _stamp(src)
    if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(f"$ {' '.join(cmd)}\n{res.stdout}{res.stderr}\n")
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}")
    stamp_file.write_text(stamp)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(HERE.glob("*.cu"))
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), sources))
    newest = max(o.stat().st_mtime for o in objs)
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = [NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static",
               "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args()
    print(build(ns.force, ns.verbose))
