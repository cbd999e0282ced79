"""Attention modules of the causal-linear path."""
from .attention_layer import AttentionLayer  # noqa: F401
from .causal_linear_attention import CausalLinearAttention, causal_linear  # noqa: F401
