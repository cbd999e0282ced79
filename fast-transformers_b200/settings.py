"""Process-wide arithmetic mode of the causal product.

The reference's ``"causal-linear"`` registry entry has no parameter for the arithmetic, and
its signature must stay unchanged, so the choice lives here: a module-level setting, a
context manager, or the environment variable ``FTB200_MODE`` read at import.

* ``"fp32"`` -- fp32 FMA on CUDA cores; matches an fp64 oracle to <= 1e-5 (relative to the
  largest magnitude of the result).  Default.
* ``"mma"``  -- tcgen05 tensor cores (TF32 operands for fp32 tensors, bf16 operands for bf16
  tensors), fp32 accumulation and fp32 running state; <= 2e-2 on the same metric.
* ``"tf32x3"`` -- the accuracy of ``"fp32"`` on the tensor cores: every fp32 operand is split into
  a TF32-exact high part and a low part and every product becomes three (fp32 accumulation);
  <= 1e-5.  The split-operand kernels take the causal product and its backward for fp32 tensors
  with 64-wide queries and values; every other shape, and every other operation, runs as in
  ``"fp32"`` (the same accuracy tier).
"""
import contextlib
import os
import threading

_MODES = ("fp32", "mma", "tf32x3")
_default = os.environ.get("FTB200_MODE", "fp32").lower()
if _default not in _MODES:
    raise ValueError("FTB200_MODE must be one of %r, got %r" % (_MODES, _default))
_local = threading.local()


def get_mode():
    """Mode used by calls made from this thread."""
    return getattr(_local, "mode", None) or _default


def set_mode(name):
    """Set the process-wide default mode."""
    global _default
    if name not in _MODES:
        raise ValueError("mode must be one of %r, got %r" % (_MODES, name))
    _default = name


@contextlib.contextmanager
def mode(name):
    """Use ``name`` for calls made by this thread inside the ``with`` block.  The mode in
    force during the forward pass is recorded for its backward pass, which autograd runs on
    another thread."""
    if name not in _MODES:
        raise ValueError("mode must be one of %r, got %r" % (_MODES, name))
    prev = getattr(_local, "mode", None)
    _local.mode = name
    try:
        yield
    finally:
        _local.mode = prev
