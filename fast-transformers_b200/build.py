"""Build recipe of the native library ``libftb200.so`` (in-tree, next to this file).

``nvcc`` cross-compiles for sm_100a without a GPU, so this runs on any machine that has the
CUDA 12.9 toolkit.  The library is a plain C-ABI shared object (``include/ftb200.h``); it
links the CUDA runtime statically and has no dependency on torch or Python.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libftb200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def nvcc_path():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA 12.9 toolkit is required to build libftb200.so")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def dependencies():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(ROOT, "include", "ftb200.h"))
    return deps


def is_current():
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(d) <= t for d in dependencies() if os.path.exists(d))


def build(force=False, verbose=False, extra_flags=()):
    """Compile every ``.cu`` under ``csrc/`` into ``libftb200.so``; returns its path."""
    if not force and is_current():
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS, *extra_flags, "-I", os.path.join(ROOT, "include"), "-I", CSRC,
           "-o", LIB, *sources(), "-lcuda"]
    env = dict(os.environ)
    # the image's default host compiler lacks some runtime pieces; use the system one
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd, env=env)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True,
          extra_flags=["-Xptxas", "-v"] if "--ptxas" in sys.argv else [])
    print(LIB)
