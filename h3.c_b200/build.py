#!/usr/bin/env python3
"""Compile libh3b200.so for sm_100a with nvcc (in-tree, no JIT cache).

    python h3.c_b200/build.py            # build if sources changed
    python h3.c_b200/build.py --force
    python h3.c_b200/build.py --verbose  # also print ptxas register / shared-memory usage
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libh3b200.so"
NVCC = os.environ.get("NVCC", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
         "--expt-relaxed-constexpr"]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > stamp for d in deps)


def compile_one(src: Path, verbose: bool) -> Path:
    obj = OBJ / (src.stem + ".o")
    headers = list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "h3b200.h"]
    if stale(obj, [src, *headers, Path(__file__)]):
        cmd = [NVCC, *ARCH, *FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        print("+", " ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.stdout.strip():
            print(res.stdout)
        if res.stderr.strip():
            print(res.stderr, file=sys.stderr)
        if res.returncode:
            raise RuntimeError(f"nvcc failed on {src.name}")
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    if force:
        for o in OBJ.glob("*.o"):
            o.unlink()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(lambda s: compile_one(s, verbose), sources()))
    if force or stale(LIB, objects):
        cmd = [NVCC, *ARCH, "-shared", "-o", str(LIB), *map(str, objects)]
        print("+", " ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
