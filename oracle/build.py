"""Compile the C restatement of the GLA recurrence (oracle/gla_oracle.c) into
oracle/_build/libgla_oracle.so.  Test infrastructure only.

    python -m oracle.build
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "gla_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libgla_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", "-O3", "-march=native", "-fopenmp", "-fno-fast-math", "-shared", "-fPIC",
           "-o", OUT, SRC, "-lm"]
    try:
        subprocess.run(cmd, check=True, capture_output=True, text=True)
    except subprocess.CalledProcessError as e:  # pragma: no cover - toolchain problem
        raise RuntimeError(f"oracle build failed: {' '.join(cmd)}\n{e.stderr}") from e
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
