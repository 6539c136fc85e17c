"""Builds every ``csrc/*.cu`` for sm_100a into ``system_lab_b200/lib/libslab_kernels.so``.

Plain ``nvcc`` (no torch headers): the kernels export a C ABI and Python calls them through
``ctypes`` with raw device pointers and the current stream, so a rebuild takes seconds and the
library has no ABI tie to a torch version.  Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libslab_kernels.so"
OBJ_DIR = CSRC / "build"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header() -> float:
    return max((p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))), default=0.0)


def build(verbose: bool = False, force: bool = False) -> Path:
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    hdr = _newest_header()
    jobs = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ_DIR / (src.stem + ".ptxas.log")).write_text(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr[-4000:]}")
        return src.name

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for name in ex.map(compile_one, jobs):
                if verbose:
                    print(f"compiled {name}", file=sys.stderr)
    objs = [str(OBJ_DIR / (s.stem + ".o")) for s in sources]
    if jobs or not LIB.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB), *objs, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
