"""Self attention as a recurrent module: one query / key / value per call, attending to
everything seen so far (``fast_transformers/recurrent/attention/self_attention/__init__.py``)."""
from .attention_layer import RecurrentAttentionLayer  # noqa: F401
from .linear_attention import RecurrentLinearAttention  # noqa: F401
