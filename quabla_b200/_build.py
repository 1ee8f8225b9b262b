"""Builds libqb200.so in-tree with nvcc for sm_100a.

Run as ``python -m quabla_b200._build`` (add ``--force`` to rebuild, ``-v`` to
print ptxas resource usage).  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
# QB200_LIBRARY points the binding at another build of the same sources (A/B comparisons on one GPU box).
LIBRARY = os.environ.get("QB200_LIBRARY") or os.path.join(_HERE, "libqb200.so")
SOURCES = ["api.cu", "plan.cu", "static_scratch.cu", "fused.cu", "tc_gemm.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc was not found; set NVCC or put it on PATH")


def _stale() -> bool:
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    roots = [CSRC, os.path.join(os.path.dirname(_HERE), "include")]
    for root in roots:
        for name in os.listdir(root):
            if os.path.getmtime(os.path.join(root, name)) > built:
                return True
    return False


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if a source is newer than it; returns its path."""
    if not force and not _stale():
        return LIBRARY
    objects = []
    build_dir = os.path.join(_HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    common = [
        _nvcc(), *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC",
    ]
    common += os.environ.get("QB200_NVCC_FLAGS", "").split()
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for source in SOURCES:
        obj = os.path.join(build_dir, source.replace(".cu", ".o"))
        objects.append(obj)
        procs.append(subprocess.Popen(common + ["-c", os.path.join(CSRC, source), "-o", obj]))
    for proc in procs:
        if proc.wait() != 0:
            raise RuntimeError("nvcc failed")
    subprocess.check_call([_nvcc(), *ARCH_FLAGS, "-shared", "-o", LIBRARY, *objects, "-ldl"])
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
