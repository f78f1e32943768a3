"""Build the CPU oracle (test infrastructure) and, when the reference tree is
mounted, the reference's own CUDA kernels.

* ``oracle/liboracle.so``  <- ``oracle/shainet_oracle.cpp`` with
  ``g++ -O2 -ffp-contract=off -fopenmp`` (no fast-math: the sequential fp32 sums
  must stay sequential and unfused).
* ``oracle/_ref/libshainet_cuda_kernels.so`` <- the reference's single CUDA
  source, compiled unmodified from where it lies for plain ``sm_100`` (the
  arch its own build script would pick).  Only the built library lands in this
  repository's tree (git-ignored); no reference source is copied.

Run:  python oracle/build_oracle.py [reference_root]
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libshainet_cuda_kernels.so")
REF_CU_REL = os.path.join("src", "shainet", "native", "cuda_kernels.cu")


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "shainet_oracle.cpp")
    if not force and _newer(ORACLE_SO, src):
        return ORACLE_SO
    cmd = ["g++", "-O2", "-ffp-contract=off", "-fopenmp", "-fPIC", "-shared", "-std=c++17",
           "-o", ORACLE_SO, src]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_reference_kernels(reference_root: str | None = None, force: bool = False) -> str | None:
    """Compile the reference's CUDA file; returns the .so path, or None when the
    reference tree is not mounted (the prebuilt .so, if any, is then used)."""
    # the argument, else $SHAINET_REFERENCE_ROOT, else a checkout named "reference" beside this repository
    reference_root = (reference_root or os.environ.get("SHAINET_REFERENCE_ROOT")
                      or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
    src = os.path.join(reference_root, REF_CU_REL)
    if not os.path.exists(src):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, src):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-O3", "-arch=sm_100", "-shared", "-Xcompiler", "-fPIC", "-o", REF_SO, src, "-lcurand"]
    subprocess.run(cmd, check=True)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force=True))
    print(build_reference_kernels(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
