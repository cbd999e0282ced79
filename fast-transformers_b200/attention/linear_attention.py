"""Unmasked linear attention, O(L D M) per head.

Mirror of ``fast_transformers/attention/linear_attention.py``: ``LinearAttention`` (:18-80) with
the same constructor and ``forward`` arguments and the ``"linear"`` registry entry with the same
parameter tuple (:85-92).

    Q = phi(queries); K = phi(keys) * key_length_mask
    out_i = (Q_i . sum_j K_j^T V_j) / (Q_i . sum_j K_j + eps)

The numerator is the degenerate case of the causal product -- one state for the whole sequence,
no mask -- and runs on the same kernels (``causal_product.linear_product``): the reference's two
einsums over (N, L, H, .) tensors become a state sum and one pass that applies it, both reading
the (N, L, H, .) storage through strides; the default feature map and the key-length mask are
one native pass.  The denominator is a vector per head and stays a pair of torch calls.
"""
import torch
from torch.nn import Module

from ..attention_registry import (AttentionRegistry, Callable, EventDispatcherInstance, Int,
                                  Optional)
from ..causal_product.linear_product import linear_dot_product
from ..events import EventDispatcher
from ..feature_maps import elu_feature_map, elu_plus_one_native, is_default_elu_map


class LinearAttention(Module):
    """Arguments (unchanged from the reference)
    ---------
        query_dimensions: int, the dimensionality of queries and keys per head
        feature_map: callable, a FACTORY called with ``query_dimensions`` that returns the
                     feature map (default: elu(x)+1)
        eps: float, added to the denominator (default: 1e-6)
        event_dispatcher: str or EventDispatcher instance (default: the global dispatcher)
    """

    def __init__(self, query_dimensions, feature_map=None, eps=1e-6, event_dispatcher=""):
        super().__init__()
        self.feature_map = (feature_map(query_dimensions) if feature_map
                            else elu_feature_map(query_dimensions))
        self.eps = eps
        self.event_dispatcher = EventDispatcher.get(event_dispatcher)

    def forward(self, queries, keys, values, attn_mask, query_lengths, key_lengths):
        self.feature_map.new_feature_map(queries.device)
        if not attn_mask.all_ones:
            raise RuntimeError("LinearAttention does not support arbitrary attention masks")
        if (is_default_elu_map(self.feature_map) and queries.is_cuda
                and queries.dtype in (torch.float32, torch.bfloat16)):
            Q = elu_plus_one_native(queries)
            K = elu_plus_one_native(keys, key_lengths.float_matrix)
        else:
            Q = self.feature_map.forward_queries(queries)
            K = self.feature_map.forward_keys(keys)
            K = K * key_lengths.float_matrix[:, :, None, None]
        # (N, L, H, .) storage viewed as (N, H, L, .): the kernels read and write through strides
        num = linear_dot_product(Q.permute(0, 2, 1, 3), K.permute(0, 2, 1, 3),
                                 values.permute(0, 2, 1, 3)).permute(0, 2, 1, 3)
        Z = 1 / (torch.einsum("nlhd,nhd->nlh", Q, K.sum(dim=1)) + self.eps)
        return (num * Z[:, :, :, None]).contiguous()


AttentionRegistry.register(
    "linear", LinearAttention,
    [
        ("query_dimensions", Int),
        ("feature_map", Optional(Callable)),
        ("event_dispatcher", Optional(EventDispatcherInstance, ""))
    ]
)
