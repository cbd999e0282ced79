"""Causal linear attention as a recurrent model (mirror of ``fast_transformers/recurrent``
restricted to the linear self-attention step)."""
