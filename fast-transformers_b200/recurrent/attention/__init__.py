"""Autoregressive attention modules (``fast_transformers/recurrent/attention/__init__.py``): the
linear self-attention step only."""
from .self_attention.linear_attention import RecurrentLinearAttention  # noqa: F401
