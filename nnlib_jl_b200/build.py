"""Build libnnlib_b200.so in-tree with nvcc for sm_100a.

``python -m nnlib_jl_b200.build`` (or :func:`build`) compiles every ``.cu``
under ``csrc/`` to an object file and links them into
``nnlib_jl_b200/libnnlib_b200.so``.  Objects are rebuilt only when a source or
header is newer.  nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libnnlib_b200.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libnnlib_b200.so cannot be built")
    return exe


def _newest_dep_mtime() -> float:
    deps = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE_DIR.glob("*.h"))
    return max(p.stat().st_mtime for p in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile and link; returns the path of the shared library."""
    BUILD_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(CSRC.glob("*.cu"))
    dep_time = _newest_dep_mtime()
    jobs = []
    objs = []
    for src in sources:
        obj = BUILD_DIR / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, dep_time)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE_DIR), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(4, len(jobs))) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out, file=sys.stderr)
    relink = bool(jobs) or not LIB_PATH.exists() or any(o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs)
    if relink:
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH),
               *map(str, objs), "-cudart", "static"]
        run(cmd)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
