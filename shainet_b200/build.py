"""Build libshainet_attn.so (sm_100a only) in-tree with nvcc.

    python -m shainet_b200.build [--force] [--verbose]

The library links the CUDA runtime statically and nothing else: no torch, no
CUTLASS at run time.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libshainet_attn.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps() -> list[str]:
    return sources() + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        glob.glob(os.path.join(INCLUDE, "*.h"))


def up_to_date() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    t = os.path.getmtime(LIB_PATH)
    return all(os.path.getmtime(d) <= t for d in _deps())


def compile_library(out_path: str, obj_dir: str, srcs: list[str], verbose: bool = False,
                    include_dirs: list[str] | None = None) -> str:
    """nvcc every source for sm_100a (in parallel) and link them into one shared library."""
    os.makedirs(os.path.dirname(out_path), exist_ok=True)
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    common = [nvcc, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-diag-suppress", "177", "-Xcompiler", "-fPIC",
              "-I", INCLUDE]
    for d in include_dirs or []:
        common += ["-I", d]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs, objs = [], []
    for src in srcs:
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        procs.append((src, subprocess.Popen(common + ["-c", src, "-o", obj], stdout=subprocess.PIPE,
                                            stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if out.strip() and (verbose or p.returncode != 0):
            print(f"--- {os.path.basename(src)}\n{out}")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", out_path, *objs], check=True)
    return out_path


def build(force: bool = False, verbose: bool = False) -> str:
    """Build shainet_b200/lib/libshainet_attn.so unless it is newer than every source."""
    if not force and up_to_date():
        return LIB_PATH
    return compile_library(LIB_PATH, os.path.join(PKG, "build"), sources(), verbose)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
