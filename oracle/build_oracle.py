"""Build recipe for the CPU checker (test infrastructure, never part of the product).

Compiles ``linmt_oracle.cpp`` twice with g++: an AVX2 build that runs on any recent x86-64
host and an AVX-512 build picked at load time when the host CPU has it.  Outputs go to
``oracle/_build/``.  Nothing of the reference's decoder compiles without Boost and a GPU, so there
is no build of the reference itself; what ``oracle/_ref/`` holds is the same restatement with its dense
products handed to the Eigen headers the reference project ships (``package/eigen.tar.gz``, the
library its host-side beam code is written with): the build that is TIMED as the CPU baseline.  It is
made only where the reference tree is present; elsewhere the prebuilt files are used as they are.
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


REF_OUT = os.path.join(HERE, "_ref")
EIGEN_TARBALL = os.path.join(os.sep, "root", "reference", "package", "eigen.tar.gz")


def ref_lib_path(variant: str) -> str:
    return os.path.join(REF_OUT, f"liblinmt_oracle_eigen_{variant}.so")


def build_ref(force: bool = False) -> bool:
    """Eigen-GEMM build of the restatement into oracle/_ref/ (headers unpacked from the reference's own
    tarball, never copied into the repository's history).  Returns False where the tarball is absent."""
    if not os.path.exists(EIGEN_TARBALL):
        return False
    os.makedirs(REF_OUT, exist_ok=True)
    inc = os.path.join(REF_OUT, "eigen")
    if not os.path.isdir(inc):
        subprocess.run(["tar", "-xzf", EIGEN_TARBALL, "-C", REF_OUT], check=True)
    src = os.path.join(HERE, "linmt_oracle.cpp")
    for v, flag in VARIANTS.items():
        out = ref_lib_path(v)
        if not force and os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
            continue
        cmd = ["g++", "-std=c++17", "-O3", flag, "-fopenmp", "-shared", "-fPIC", "-w", "-DLINMT_ORACLE_EIGEN", "-I" + inc,
               "-o", out, src]
        subprocess.run(cmd, check=True)
    return True


def build(force: bool = False) -> None:
    build_ref(force)
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
