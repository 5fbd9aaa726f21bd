"""Build libgla_b200.so in-tree with nvcc for sm_100a.

    python -m gtr_b200.build [--force]
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
SRC_DIR = os.path.join(PKG, "csrc")
SOURCES = [os.path.join(SRC_DIR, "gla_b200.cu")]
HEADERS = [os.path.join(SRC_DIR, "gla_kernel.cuh"), os.path.join(SRC_DIR, "gla_device.cuh"),
           os.path.join(SRC_DIR, "gla_trace.cuh"),
           os.path.join(SRC_DIR, "swiglu_dwconv.cuh"), os.path.join(SRC_DIR, "gla_bwd.cuh"),
           os.path.join(ROOT, "include", "gla_b200.h")]
OUT = os.path.join(PKG, "libgla_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include")]


def nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def up_to_date() -> bool:
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    return all(os.path.getmtime(p) <= t for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return OUT
    cmd = [nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", OUT, *SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
