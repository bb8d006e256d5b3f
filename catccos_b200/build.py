"""Builds libcatccos_b200.so (the CUDA kernels and the C ABI) in-tree with nvcc for sm_100a.

    python -m catccos_b200.build            the product library
    python -m catccos_b200.build --trace    libcatccos_b200_trace.so as well: the same sources with
                                            -DCATCCOS_TRACE (device-side timeline, csrc/trace.cuh)
"""
from __future__ import annotations

import os
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libcatccos_b200.so")
TRACE_LIB_PATH = os.path.join(_HERE, "libcatccos_b200_trace.so")
SOURCES = ["capi.cu"]
INCLUDE = os.path.join(_HERE, "..", "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _inputs():
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".hpp", ".h"))]
    files += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    return files


def _stale(lib: str) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    return any(os.path.getmtime(f) > t for f in _inputs())


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Compiles the library when a source or header is newer than it (or always with force)."""
    nvcc = os.environ.get("NVCC", "nvcc")
    extra = ["-Xptxas", "-v"] if verbose else []
    if force or _stale(LIB_PATH):
        subprocess.check_call([nvcc] + NVCC_FLAGS + extra + ["-o", LIB_PATH] + SOURCES, cwd=CSRC)
    if trace and (force or _stale(TRACE_LIB_PATH)):
        subprocess.check_call([nvcc] + NVCC_FLAGS + extra + ["-DCATCCOS_TRACE=1", "-o", TRACE_LIB_PATH] + SOURCES, cwd=CSRC)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
