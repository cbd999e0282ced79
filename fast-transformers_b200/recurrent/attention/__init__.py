"""Autoregressive attention modules (``fast_transformers/recurrent/attention/__init__.py``): the
linear self-attention step and the projection layer around it."""
from .self_attention.attention_layer import RecurrentAttentionLayer  # noqa: F401
from .self_attention.linear_attention import RecurrentLinearAttention  # noqa: F401
from .cross_attention.linear_attention import RecurrentCrossLinearAttention  # noqa: F401
