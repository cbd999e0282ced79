"""B200-native causal linear attention: a drop-in for the causal linear-attention path of
fast-transformers (``fast_transformers.causal_product`` and
``fast_transformers.attention.causal_linear_attention``).

Layout of the package (mirrors the reference's module names for this path only):

* ``causal_product``      -- ``causal_dot_product`` / ``CausalDotProduct`` (autograd Function)
  over the native C-ABI library ``libftb200.so`` (CUDA kernels for sm_100a).
* ``attention``           -- ``CausalLinearAttention`` and the ``AttentionLayer`` wrapper.
* ``attention_registry``  -- the plugin table holding the ``"causal-linear"`` entry.
* ``feature_maps``        -- ``elu_feature_map`` and ``Favor``.
* ``masking``, ``events``, ``builders``, ``transformers`` -- the small host-side pieces an
  encoder built with ``attention_type="causal-linear"`` needs.
* ``sequence_parallel``   -- a sequence split across ranks with one exchange of states.

There is no CPU implementation and no fallback: CUDA tensors on a B200 are required and a
missing native library raises at the first call.
"""
__version__ = "0.1.0"

from . import _native  # noqa: F401  (defines the loader; loads lazily)
from .settings import get_mode, set_mode, mode  # noqa: F401


def check_device_status(device=None, reset=True):
    """Wait for ``device`` (default: the current CUDA device) to finish everything queued on it
    and raise ``_native.NativeError`` if one of this library's kernels recorded an error there:
    every device-side wait in the kernels is bounded, and a wait that runs out (a peer GPU that
    never delivers, a broken pipeline) leaves ``FTB_ERR_TIMEOUT`` in a status word instead of
    hanging.  The product calls do not synchronise, so they cannot report it themselves; call
    this where the program synchronises anyway -- at the end of a step, before results are
    trusted.  ``reset`` clears the word."""
    import torch
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _native.check(_native.lib().ftb_device_status(int(bool(reset))), "a kernel of this library")
