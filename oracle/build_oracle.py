"""Build recipe for the CPU checker (test infrastructure, never part of the product).

Compiles ``linmt_oracle.cpp`` twice with g++: an AVX2 build that runs on any recent x86-64
host and an AVX-512 build picked at load time when the host CPU has it.  Outputs go to
``oracle/_build/``.  Nothing of the reference compiles without Boost and a GPU, so there is
no ``oracle/_ref`` build of the reference itself.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")
VARIANTS = {"v3": "-march=x86-64-v3", "v4": "-march=x86-64-v4"}


def lib_path(variant: str) -> str:
    return os.path.join(OUT, f"liblinmt_oracle_{variant}.so")


def build(force: bool = False) -> None:
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "linmt_oracle.cpp")
    for v, flag in VARIANTS.items():
        out = lib_path(v)
        if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
            continue
        cmd = ["g++", "-std=c++17", "-O3", flag, "-fopenmp", "-shared", "-fPIC", "-o", out, src]
        subprocess.run(cmd, check=True)


if __name__ == "__main__":
    build(force="--force" in sys.argv)
    print("built", [lib_path(v) for v in VARIANTS])
