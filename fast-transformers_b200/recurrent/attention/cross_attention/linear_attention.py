"""Unmasked linear attention over a fixed memory, one query per call.

Mirror of ``fast_transformers/recurrent/attention/cross_attention/linear_attention.py:18-79``:
same constructor, same ``forward(query, keys, values, key_lengths, state=None)``, same registry
entry ``"linear"`` in the recurrent cross-attention registry (:83-90).  On the first call the
state is built from the memory -- ``S = sum_s K_s (x) v_s`` by ``ftb_causal_state_sum`` over the
(N, S, H, .) storage, ``z = sum_s K_s`` -- and every call is then one read-only launch,
``y = (Q . S) / (Q . z + eps)`` (``ftb_recurrent_cross_linear_step``; the reference: two einsums
and a reciprocal, :66-69), with ``elu(x) + 1`` applied to the query inside the kernel for the
default feature map.

The state is returned as ``[S, z]`` with ``S`` shaped (N, H, M, D) as in the reference (:61); here
that is a transposed view of the (N, H, D, M) float32 block the kernels read.  CUDA tensors only;
inference only (a call that would record gradients raises).
"""
import ctypes

import torch
from torch.nn import Module

from .... import _native
from ....attention_registry import (Callable, EventDispatcherInstance, Int, Optional,
                                    RecurrentCrossAttentionRegistry)
from ....causal_product import causal_state_sum
from ....events import EventDispatcher
from ....feature_maps import elu_feature_map, elu_plus_one_native, is_default_elu_map


def recurrent_cross_linear_step(Q, S, z, eps=1e-6, elu_plus_one=False):
    """``y = (phi(Q) . S) / (phi(Q) . z + eps)`` for (N, H, D) queries (features already unless
    ``elu_plus_one``), float32 contiguous ``S`` (N, H, D, M) and ``z`` (N, H, D); nothing is
    modified.  Returns (N, H, M)."""
    for t in (Q, S, z):
        if not t.is_cuda:
            raise RuntimeError("recurrent_cross_linear_step needs CUDA tensors (there is no CPU path)")
    if Q.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("the query must be float32 or bfloat16")
    N, H, D = Q.shape
    if S.dtype != torch.float32 or z.dtype != torch.float32 or not S.is_contiguous() or not z.is_contiguous():
        raise RuntimeError("the state must be contiguous float32 tensors")
    if S.shape[:3] != (N, H, D) or z.shape != (N, H, D):
        raise RuntimeError("the state does not match the query")
    M = S.shape[3]
    Q = Q if Q.stride(-1) == 1 or D <= 1 else Q.contiguous()
    out = torch.empty(N, H, M, device=Q.device, dtype=Q.dtype)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())   # noqa: E731
    with torch.cuda.device(Q.device):
        st = _native.lib().ftb_recurrent_cross_linear_step(
            ptr(Q), ptr(S), ptr(z), ptr(out), N, H, D, M, _native.strides2(Q), _native.strides2(out),
            0 if Q.dtype == torch.float32 else 1,
            _native.FEATURE_ELU1 if elu_plus_one else _native.FEATURE_NONE, float(eps),
            ctypes.c_void_p(torch.cuda.current_stream(Q.device).cuda_stream))
    _native.check(st, "ftb_recurrent_cross_linear_step")
    return out


class RecurrentCrossLinearAttention(Module):
    """Arguments (unchanged from the reference)
    ---------
        query_dimensions: int, the dimensionality of queries and keys per head
        feature_map: callable, a FACTORY called with ``query_dimensions`` (default: elu(x)+1)
        eps: float, added to the denominator (default: 1e-6)
        event_dispatcher: str or EventDispatcher instance (default: the global dispatcher)
    """

    def __init__(self, query_dimensions, feature_map=None, eps=1e-6, event_dispatcher=""):
        super().__init__()
        self.feature_map = (feature_map(query_dimensions) if feature_map
                            else elu_feature_map(query_dimensions))
        self.eps = eps
        self.event_dispatcher = EventDispatcher.get(event_dispatcher)

    def memory_state(self, keys, values, key_lengths):
        """``[S, z]`` of a memory: keys (N, S, H, D), values (N, S, H, M), ``key_lengths`` a
        length mask; S as an (N, H, M, D) view, z (N, H, D), both float32."""
        default = is_default_elu_map(self.feature_map) and keys.dtype in (torch.float32, torch.bfloat16)
        if default:
            K = elu_plus_one_native(keys, key_lengths.float_matrix)
        else:
            K = self.feature_map.forward_keys(keys) * key_lengths.float_matrix[:, :, None, None]
        S = causal_state_sum(K.permute(0, 2, 1, 3), values.to(K.dtype).permute(0, 2, 1, 3))
        z = K.sum(dim=1, dtype=torch.float32).contiguous()
        return [S.transpose(2, 3), z]

    def forward(self, query, keys, values, key_lengths, state=None):
        if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (query, keys, values)):
            raise RuntimeError("RecurrentCrossLinearAttention is inference only here; use "
                               "LinearAttention (the batch form) to train")
        if state is None:
            self.feature_map.new_feature_map(query.device)
            state = self.memory_state(keys, values, key_lengths)
        S_ref, z = state
        S = S_ref.transpose(2, 3)           # (N, H, D, M); contiguous when it came from memory_state
        if not S.is_contiguous() or S.dtype != torch.float32:
            S = S.float().contiguous()
        z = z if (z.dtype == torch.float32 and z.is_contiguous()) else z.float().contiguous()
        default = is_default_elu_map(self.feature_map) and query.dtype in (torch.float32, torch.bfloat16)
        Q = query if default else self.feature_map.forward_queries(query)
        y = recurrent_cross_linear_step(Q, S, z, self.eps, elu_plus_one=default)
        return y, [S_ref, z]


RecurrentCrossAttentionRegistry.register(
    "linear", RecurrentCrossLinearAttention,
    [
        ("query_dimensions", Int),
        ("feature_map", Optional(Callable)),
        ("event_dispatcher", Optional(EventDispatcherInstance, ""))
    ]
)
