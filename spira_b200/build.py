"""Builds ``libspira_b200.so`` (the C-ABI library declared in ``include/spira_b200.h``) in-tree.

Plain nvcc calls, sm_100a only:  python -m spira_b200.build [--force]
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libspira_b200.so"
SOURCES = ["api.cu", "keys.cu", "ingest.cu", "kmap.cu", "group.cu", "pointwise.cu", "conv.cu", "dense.cu", "tape.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-I", str(INCLUDE), "-I", str(CSRC)]


def _newest_input() -> float:
    files = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")) + [Path(__file__)]
    return max(f.stat().st_mtime for f in files)


def build(force: bool = False, verbose: bool = False) -> Path:
    if LIB.exists() and not force and LIB.stat().st_mtime > _newest_input():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)

    def one(src: str) -> Path:
        obj = objdir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    with cf.ThreadPoolExecutor(len(SOURCES)) as ex:
        objs = list(ex.map(one, SOURCES))
    r = subprocess.run([nvcc, "-shared", "-o", str(LIB), *[str(o) for o in objs]], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
