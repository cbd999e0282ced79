"""The multi-head projections around a recurrent attention step.

Mirror of ``fast_transformers/recurrent/attention/self_attention/attention_layer.py:15-97``
(``RecurrentAttentionLayer``): the same four ``Linear`` layers under the same attribute names as
``AttentionLayer``, so a state dict of the batch model loads into the recurrent one; ``forward``
projects ONE position (N, D), splits it into heads and calls the inner attention with the state.

Added here: ``prefill`` -- a whole prefix (N, L, D) in batch form through the same weights, which
returns the state the steps continue from (the reference would loop over the prefix).
"""
from torch.nn import Linear, Module

from ....events import EventDispatcher
from ..._utils import check_state


class RecurrentAttentionLayer(Module):
    """Arguments (as in the reference, ``attention_layer.py:22-36``)
    ---------
        attention: the inner recurrent attention (``forward(query, key, value, state)``)
        d_model: int, the input feature dimensionality
        n_heads: int
        d_keys, d_values: int, per-head dimensions (default: d_model // n_heads)
        d_model_keys: int, dimensionality of the inputs keys and values are projected from
                      (default: d_model)
        event_dispatcher: str or EventDispatcher instance
    """

    def __init__(self, attention, d_model, n_heads, d_keys=None, d_values=None,
                 d_model_keys=None, event_dispatcher=""):
        super(RecurrentAttentionLayer, self).__init__()
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

    def forward(self, query, key, value, state=None, memory=None):
        """query, key, value: (N, D), one position.  Returns (new value (N, D), state)."""
        state = check_state(state, memory)
        N, H = query.shape[0], self.n_heads
        new_value, state = self.inner_attention(
            self.query_projection(query).view(N, H, -1),
            self.key_projection(key).view(N, H, -1),
            self.value_projection(value).view(N, H, -1),
            state)
        return self.out_projection(new_value.reshape(N, -1)), state

    def prefill(self, query, key, value, key_lengths=None):
        """query, key, value: (N, L, D), a whole prefix.  Returns the new values (N, L, D) -- what
        the batch ``AttentionLayer`` with these weights gives under a causal mask -- and the state
        after position L-1 (after each sequence's last valid position with ``key_lengths``)."""
        N, L, H = query.shape[0], query.shape[1], self.n_heads
        new_values, state = self.inner_attention.prefill(
            self.query_projection(query).view(N, L, H, -1),
            self.key_projection(key).view(N, L, H, -1),
            self.value_projection(value).view(N, L, H, -1),
            key_lengths)
        return self.out_projection(new_values.reshape(N, L, -1)), state
