"""Attention modules of the linear-attention path: the causal layer and its unmasked form."""
from .attention_layer import AttentionLayer  # noqa: F401
from .causal_linear_attention import CausalLinearAttention, causal_linear  # noqa: F401
from .linear_attention import LinearAttention  # noqa: F401
