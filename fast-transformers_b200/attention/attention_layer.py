"""Multi-head wrapper: project to heads, run the inner attention, project back.

Mirror of ``fast_transformers/attention/attention_layer.py:21-115`` (same constructor,
same ``forward(queries, keys, values, attn_mask, query_lengths, key_lengths)``, same
parameter names ``query_projection`` / ``key_projection`` / ``value_projection`` /
``out_projection`` so state dicts interchange).  The four projections are library GEMMs.
"""
from torch.nn import Linear, Module

from ..events import EventDispatcher, QKVEvent


class AttentionLayer(Module):
    def __init__(self, attention, d_model, n_heads, d_keys=None, d_values=None,
                 d_model_keys=None, event_dispatcher=""):
        super().__init__()
        d_keys = d_keys or (d_model // n_heads)
        d_values = d_values or (d_model // n_heads)
        d_model_keys = d_model_keys or d_model
        self.inner_attention = attention
        self.query_projection = Linear(d_model, d_keys * n_heads)
        self.key_projection = Linear(d_model_keys, d_keys * n_heads)
        self.value_projection = Linear(d_model_keys, d_values * n_heads)
        self.out_projection = Linear(d_values * n_heads, d_model)
        self.n_heads = n_heads
        self.event_dispatcher = EventDispatcher.get(event_dispatcher)

    def forward(self, queries, keys, values, attn_mask, query_lengths, key_lengths):
        """queries (N, L, d_model), keys/values (N, S, d_model_keys) -> (N, L, d_model)."""
        N, L, _ = queries.shape
        S = keys.shape[1]
        H = self.n_heads
        queries = self.query_projection(queries).view(N, L, H, -1)
        keys = self.key_projection(keys).view(N, S, H, -1)
        values = self.value_projection(values).view(N, S, H, -1)
        self.event_dispatcher.dispatch(QKVEvent(self, queries, keys, values))
        new_values = self.inner_attention(
            queries, keys, values, attn_mask, query_lengths, key_lengths
        ).reshape(N, L, -1)
        return self.out_projection(new_values)
