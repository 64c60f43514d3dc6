"""Builds the CUDA library in-tree: patina_b200/_lib/libpatina_gemm.so.

nvcc cross-compiles for sm_100a without a GPU. Run as `python -m patina_b200.build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_PKG, "csrc")
LIB_DIR = os.path.join(_PKG, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libpatina_gemm.so")
HARNESS_PATH = os.path.join(LIB_DIR, "gemm_check")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.isfile(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))
               if f.endswith((".cu", ".cuh", ".h"))]
    sources.append(os.path.join(_PKG, "..", "include", "patina_gemm.h"))
    if force or _stale(LIB_PATH, sources):
        cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH, os.path.join(CSRC, "patina_gemm.cu")]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
        subprocess.check_call(cmd)
    return LIB_PATH


def build_harness(force: bool = False) -> str:
    """The C++ harness (drop-in for the reference's gemm_check CLI), linked to the library."""
    src = os.path.join(_PKG, "harness", "gemm_check.cpp")
    if not os.path.isfile(src):
        return ""
    build_library()
    if force or _stale(HARNESS_PATH, [src, LIB_PATH]):
        cxx = os.environ.get("CXX", "g++")
        subprocess.check_call([
            cxx, "-O2", "-std=c++17", "-I", os.path.join(_PKG, "..", "include"),
            "-I", "/usr/local/cuda/include", src, "-o", HARNESS_PATH,
            "-L", LIB_DIR, "-lpatina_gemm", "-Wl,-rpath,$ORIGIN",
            "-L", "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64",
            "-lpthread", "-ldl", "-lm",
        ])
    return HARNESS_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    h = build_harness(force="--force" in sys.argv)
    if h:
        print(h)
