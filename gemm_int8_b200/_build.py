"""Builds libgemm_int8_b200.so in-tree with nvcc for sm_100a (no libtorch, no CUTLASS).

Replaces the reference's CMake/ninja build of gemm_int8_CUDA.so (CMakeLists.txt, build.sh): one
translation unit, one nvcc command, a few seconds.
"""
from __future__ import annotations

import os
import shutil
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libgemm_int8_b200.so"
LIB_PATH = os.path.join(_PKG, LIB_NAME)
SOURCES = [os.path.join(_PKG, "csrc", "api.cu")]
HEADERS = [os.path.join(_PKG, "csrc", f) for f in ("ptx.cuh", "k_dense.cuh", "k_dense_splitk.cuh", "k_blockwise.cuh", "k_smallm.cuh", "k_quant.cuh")]
HEADERS.append(os.path.join(os.path.dirname(_PKG), "include", "gemm_int8_b200.h"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build " + LIB_NAME)
    return cand


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.exists(f) and os.path.getmtime(f) > t for f in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, *SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True, verbose=True))
