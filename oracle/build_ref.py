"""Build recipe for the checker binaries under ``oracle/``. TEST INFRASTRUCTURE ONLY.

Two things are compiled here, both CPU-only:

1. ``oracle/_ref/causal_product_cpu.so`` -- the reference's own OpenMP extension,
   compiled *in place* from the reference checkout
   (``fast_transformers/causal_product/causal_product_cpu.cpp``) with the flags its
   ``setup.py:67-73`` uses (``-fopenmp -ffast-math``).  No reference source is copied
   into this repository; only the built object lands in ``oracle/_ref/`` (git-ignored).
   It is skipped silently when the reference checkout is not present (the prebuilt
   ``.so`` is used instead if it exists).
2. ``oracle/libcausal_oracle_c.so`` -- this repository's plain-C restatement of the same
   recurrence (``oracle/causal_oracle.c``).

Neither is ever loaded by the product path; only ``tests/``, the smoke check and the
CPU-baseline / reference arm of ``bench.py`` use them.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "causal_product_cpu.so")
C_SO = os.path.join(HERE, "libcausal_oracle_c.so")
C_SRC = os.path.join(HERE, "causal_oracle.c")

# The system compilers: the image's default CXX cannot link OpenMP.
GXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
GCC = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"


def reference_root():
    """Location of the reference checkout, or None when it is not mounted."""
    root = os.environ.get("FAST_TRANSFORMERS_REFERENCE", "/root/reference")
    src = os.path.join(root, "fast_transformers", "causal_product",
                       "causal_product_cpu.cpp")
    return root if os.path.exists(src) else None


def _newer(target, *sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_c_oracle(verbose=False):
    if _newer(C_SO, C_SRC):
        return C_SO
    cmd = [GCC, "-O2", "-fopenmp", "-shared", "-fPIC", "-o", C_SO, C_SRC, "-lm"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return C_SO


def build_reference_ext(verbose=False):
    """Compile the reference CPU extension where its source lies; returns the .so path
    or None when neither the source nor a prebuilt object is available."""
    root = reference_root()
    if root is None:
        return REF_SO if os.path.exists(REF_SO) else None
    src = os.path.join(root, "fast_transformers", "causal_product",
                       "causal_product_cpu.cpp")
    if _newer(REF_SO, src):
        return REF_SO
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(REF_DIR, exist_ok=True)
    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [GXX, "-O2", "-std=c++17", "-shared", "-fPIC", "-fopenmp", "-ffast-math",
           "-DTORCH_EXTENSION_NAME=causal_product_cpu",
           "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           *inc, src, "-o", REF_SO,
           "-L" + libdir, "-Wl,-rpath," + libdir,
           "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return REF_SO


def main():
    build_c_oracle(verbose=True)
    so = build_reference_ext(verbose=True)
    print("reference extension:", so or "not available (no reference checkout)")


if __name__ == "__main__":
    sys.exit(main())
