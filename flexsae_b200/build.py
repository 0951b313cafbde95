"""Builds the CUDA library in-tree: ``flexsae_b200/_lib/libflexsae_b200.so`` for sm_100a.

nvcc cross-compiles without a GPU, so this runs on a CPU-only machine; the shared object then
travels with the source tree.  ``python -m flexsae_b200.build`` rebuilds when a source is newer
than the library; ``--force`` always rebuilds; ``--verbose`` prints ptxas resource usage;
``--trace`` builds the tuning variant ``libflexsae_b200_trace.so`` (compiled with
``-DFLEXSAE_TRACE``: the sharded backward records a per-slot timeline, see ``slot_timeline.py``).
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libflexsae_b200.so")
TRACE_LIB_PATH = os.path.join(LIB_DIR, "libflexsae_b200_trace.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale(lib_path: str = LIB_PATH) -> bool:
    if not os.path.exists(lib_path):
        return True
    t = os.path.getmtime(lib_path)
    deps = _sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Compiles every ``csrc/*.cu`` into one shared library and returns its path."""
    out = TRACE_LIB_PATH if trace else LIB_PATH
    if not force and not _stale(out):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built on this machine")
    os.makedirs(LIB_DIR, exist_ok=True)
    extra = os.environ.get("FLEXSAE_NVCC_EXTRA", "--use_fast_math").split()   # e.g. "-DFLEXSAE_BWD_MINB=8" while tuning
    if trace:
        extra = extra + ["-DFLEXSAE_TRACE"]
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-I", INCLUDE, "-o", tmp] + _sources()
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout)
    if res.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError("nvcc failed:\n" + res.stdout[-4000:])
    os.replace(tmp, out)    # a reader (another rank, a running job) never sees a half-written library
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
