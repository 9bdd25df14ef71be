"""Build libgptb200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Usage:  python -m gpt_b200.build [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The shared object lands in gpt_b200/lib/ next to the
sources so that it is found by gpt_b200.load_library() without any install step.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libgptb200.so")
BACKEND_LIB = os.path.join(LIBDIR, "libgptb200_backend.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libgptb200.so cannot be built")
    return exe


def _sources(*names: str) -> list[str]:
    return [os.path.join(CSRC, n) for n in names]


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False, out: str | None = None, defines: list[str] | None = None) -> str:
    """`out` / `defines`: build a variant of the library somewhere else with extra -D flags (kernel experiments)."""
    if out:
        cu = [f for f in _sources("capi.cu", "backend_capi.cu", "b200_backend.cu", "gpt_model.cu", "noalloc.cu", "loader.cpp") if os.path.exists(f)]
        cmd = [_nvcc(), "-std=c++17", "-O3", *ARCH_FLAGS, "-lineinfo", "-Xcompiler", "-fPIC", "-shared", *[f"-D{d}" for d in (defines or [])],
               "-I", os.path.join(HERE, "..", "include"), "-I", CSRC, "-I", os.path.join(CSRC, "iface"), "-o", out, *cu]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("nvcc failed building " + out)
        return out
    os.makedirs(LIBDIR, exist_ok=True)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "gptb200.h")]
    cu = _sources("capi.cu", "backend_capi.cu", "b200_backend.cu", "gpt_model.cu", "noalloc.cu", "loader.cpp")
    cu = [f for f in cu if os.path.exists(f)]
    if force or _stale(LIB, deps):
        cmd = [_nvcc(), "-std=c++17", "-O3", *ARCH_FLAGS, "-lineinfo", "-Xcompiler", "-fPIC", "-shared",
               "-I", os.path.join(HERE, "..", "include"), "-I", CSRC, "-I", os.path.join(CSRC, "iface"), "-o", LIB, *cu]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), file=sys.stderr)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed building libgptb200.so")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
