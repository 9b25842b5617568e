"""Builds ``libspira_b200.so`` (the C-ABI library declared in ``include/spira_b200.h``) in-tree.

Plain nvcc calls, sm_100a only:  python -m spira_b200.build [--force]
"""
from __future__ import annotations

import concurrent.futures as cf
import fcntl
import os
import subprocess
import sys
import time
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libspira_b200.so"
SOURCES = ["api.cu", "keys.cu", "ingest.cu", "kmap.cu", "group.cu", "pointwise.cu", "conv.cu", "dense.cu", "tape.cu"]
_T0 = time.time()          # start of this process: a forced build by a sibling after this point is not repeated
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-I", str(INCLUDE), "-I", str(CSRC)]


def _newest_input() -> float:
    files = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h")) + [Path(__file__)]
    return max(f.stat().st_mtime for f in files)


def _compile_and_link(lib: Path, objdir: Path, verbose: bool) -> None:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
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
    # link beside the target and move the finished file into place: a process that loads the library while another one
    # rebuilds it (several ranks started together) sees the old file or the new one, never a part of one
    tmp = lib.with_name(f"{lib.name}.{os.getpid()}.tmp")
    r = subprocess.run([nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs]], capture_output=True, text=True)
    if r.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)


def build(force: bool = False, verbose: bool = False, lib: Path = LIB, objdir: Path | None = None) -> Path:
    """Builds the library if it is missing or older than its sources.  Safe to call from several processes at once (the
    ranks of one node): one of them builds under a file lock, the others wait for it and find the library up to date."""
    def fresh() -> bool:
        return lib.exists() and lib.stat().st_mtime > _newest_input()

    if fresh() and not force:
        return lib
    with open(lib.with_name(lib.name + ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            # (another process may have finished the same build while this one waited; a forced build is repeated only
            # if the library is older than this call)
            if fresh() and (not force or lib.stat().st_mtime >= _T0):
                return lib
            _compile_and_link(lib, objdir if objdir is not None else PKG / "build", verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
