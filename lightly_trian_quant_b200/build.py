"""Builds the C-ABI shared library (libkf_b200.so) in-tree with nvcc for sm_100a.

    python -m lightly_trian_quant_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects are cached under csrc/build/ keyed by a hash of each source and the
shared headers, so an unchanged file is not recompiled.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libkf_b200.so"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-DKF_BUILD"]


def sources():
    return sorted(CSRC.glob("*.cu"))


def _headers_hash() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.glob("*.cuh")) + sorted((PKG.parent / "include").glob("*.h")):
        h.update(p.read_bytes())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    bdir = CSRC / "build"
    bdir.mkdir(exist_ok=True)
    hh = _headers_hash()
    jobs = []
    objs = []
    for src in sources():
        tag = hashlib.sha256(src.read_bytes() + hh.encode()).hexdigest()[:16]
        obj = bdir / f"{src.stem}.{tag}.o"
        objs.append(obj)
        if force or not obj.exists():
            for old in bdir.glob(f"{src.stem}.*.o"):
                old.unlink()
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)] + (["-Xptxas", "-v"] if verbose else [])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or force or not LIB.exists():
        cmd = [NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
