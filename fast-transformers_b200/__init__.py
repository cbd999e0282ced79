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
