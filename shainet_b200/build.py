"""Build libshainet_attn.so (sm_100a only) in-tree with nvcc.

    python -m shainet_b200.build [--force] [--verbose]
    python -m shainet_b200.build --variant NAME -DMACRO[=VALUE] ...   # lib/libshainet_attn_NAME.so (measurement builds)
    python -m shainet_b200.build --harness                             # lib/capi_timing (C program over the C ABI)

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


def build(force: bool = False, verbose: bool = False, variant: str | None = None, defines: list[str] | None = None) -> str:
    """The product library, or (variant) a measurement build of the same sources with
    extra -D macros, e.g. SK_TIMELINE (device timestamps) or SK_NOMATH (copy only)."""
    out_path = LIB_PATH if variant is None else os.path.join(LIB_DIR, f"libshainet_attn_{variant}.so")
    if variant is None and not force and up_to_date():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(PKG, "build" if variant is None else f"build_{variant}")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    common = [nvcc, *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-diag-suppress", "177", "-Xcompiler", "-fPIC",
              "-I", INCLUDE]
    common += list(defines or [])
    if verbose:
        common += ["-Xptxas", "-v"]
    procs, objs = [], []
    for src in sources():
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


def build_harness() -> str:
    """csrc/capi_timing.cpp: a C++ program that times decode through the C ABI."""
    out = os.path.join(LIB_DIR, "capi_timing")
    os.makedirs(LIB_DIR, exist_ok=True)
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.run(["g++", "-O2", "-std=c++17", "-o", out, os.path.join(CSRC, "capi_timing.cpp"), f"-I{cuda}/include",
                    f"-L{cuda}/lib64", "-lcudart", "-ldl", f"-Wl,-rpath,{cuda}/lib64"], check=True)
    return out


if __name__ == "__main__":
    if "--harness" in sys.argv:
        print(build_harness())
    elif "--variant" in sys.argv:
        name = sys.argv[sys.argv.index("--variant") + 1]
        print(build(force=True, verbose="--verbose" in sys.argv, variant=name,
                    defines=[a for a in sys.argv if a.startswith("-D")]))
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
