"""Build recipe for the reference engine's own native module (TEST INFRASTRUCTURE, not product).

Compiles the reference's C++/CUDA sources *where they lie* (a read-only checkout whose
location is given by --src or the SPIRA_REF_SRC environment variable) with plain nvcc
calls and links them into ``oracle/_ref/_C.so`` -- the pybind11 module the reference's
Python shim imports as ``spira.nn.functional._C``.  No reference source is copied; only
object files and the final shared object are written, all under ``oracle/_ref/``.
The reference's CMake build is not run: this script is the whole recipe.

The reference's Python package (``source/spira``) and its model definitions
(``scripts/models/spira``) are staged next to the module, under ``oracle/_ref/spira`` and
``oracle/_ref/models``, so that the reference's own Python can drive its module on the GPU
box, where the checkout does not exist.  ``oracle/_ref/`` is not tracked: nothing of the
reference enters the repository's history.

The resulting module runs only on a machine with a GPU.  It is used by the GPU parity
tests (kernel maps and features against the reference's own kernels) and by
``bench.py --impl reference``.
"""
import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"


def _flags(csrc: Path):
    import torch
    from torch.utils import cpp_extension as ce
    import pybind11

    inc = [str(csrc), sysconfig.get_paths()["include"], pybind11.get_include()]
    inc += ce.include_paths("cuda")
    flags = ["-std=c++17", "-O3", "-Xptxas", "-O3", "-lineinfo", "--extended-lambda",
             "--expt-relaxed-constexpr", "-w",
             "-gencode", "arch=compute_100,code=sm_100",
             "-Xcompiler", "-fPIC", "-DENABLE_CUDA", "-DTORCH_EXTENSION_NAME=_C",
             "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             "-ccbin", "/usr/bin/g++"]
    for i in inc:
        flags += ["-I", i]
    libdir = str(Path(torch.__file__).parent / "lib")
    cuda_lib = str(Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "lib64")
    link = ["-shared", "-L", libdir, "-L", cuda_lib, "-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch_python", "-lcudart", f"-Wl,-rpath,{libdir}"]
    import importlib.util
    spec = importlib.util.find_spec("nvidia.cublas")
    cublas = "-lcublas"
    if spec is not None and spec.submodule_search_locations:
        cb = Path(list(spec.submodule_search_locations)[0])
        flags += ["-I", str(cb / "include")]
        link += ["-L", str(cb / "lib"), f"-Wl,-rpath,{cb / 'lib'}"]
        # pip's cuBLAS ships only the versioned .so
        for so in sorted((cb / "lib").glob("libcublas.so*")):
            cublas = f"-l:{so.name}"
            break
    link.append(cublas)
    return flags, link


def stage_python(src: str) -> None:
    """Copies the reference's Python files (package ``spira`` and the ``models/spira`` definitions of its scripts) into
    ``oracle/_ref/`` -- an untracked directory that travels to the GPU box with the built module."""
    root = Path(src)
    for rel_src, rel_dst in (("source/spira", "spira"), ("scripts/models/spira", "models/spira")):
        a, b = root / rel_src, OUT / rel_dst
        if not a.is_dir():
            raise FileNotFoundError(f"reference Python sources not found under {a}")
        if b.exists():
            shutil.rmtree(b)
        shutil.copytree(a, b, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.so"))


def build(src: str, jobs: int = 8, force: bool = False) -> Path:
    csrc = Path(src) / "source" / "csrc"
    if not csrc.is_dir():
        raise FileNotFoundError(f"reference sources not found under {csrc}")
    OUT.mkdir(exist_ok=True)
    stage_python(src)
    target = OUT / "_C.so"
    sources = sorted(list(csrc.glob("spira/**/*.cu")) + list(csrc.glob("spira/**/*.cpp")))
    if target.exists() and not force and all(target.stat().st_mtime > s.stat().st_mtime for s in sources):
        return target
    flags, link = _flags(csrc)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

    def one(s: Path):
        obj = OUT / (s.relative_to(csrc).as_posix().replace("/", "__") + ".o")
        extra = ["-x", "cu"] if s.suffix == ".cpp" else []
        if obj.exists() and not force and obj.stat().st_mtime > s.stat().st_mtime:
            return obj
        cmd = [nvcc, *flags, *extra, "-c", str(s), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n{r.stderr[-4000:]}")
        return obj

    with cf.ThreadPoolExecutor(jobs) as ex:
        objs = list(ex.map(one, sources))
    r = subprocess.run(["/usr/bin/g++", *[str(o) for o in objs], *link, "-o", str(target)], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    for o in objs:
        o.unlink()
    return target


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=os.environ.get("SPIRA_REF_SRC", str(HERE.parents[1] / "reference")),
                    help="root of the reference checkout (default: a directory named reference beside this repository)")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.src, a.jobs, a.force))
