"""Causal linear attention as a recurrent model (mirror of ``fast_transformers/recurrent``
restricted to linear self-attention: the step, its projection layer and the encoder)."""
