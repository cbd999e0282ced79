"""Attention over a fixed memory as a recurrent module: one query per call
(``fast_transformers/recurrent/attention/cross_attention/__init__.py``)."""
from .linear_attention import RecurrentCrossLinearAttention  # noqa: F401
