"""Causally masked linear attention as a recurrent model with a fixed-size state.

Mirror of ``fast_transformers/recurrent/attention/self_attention/linear_attention.py:19-102``:
same constructor, same ``forward(query, key, value, state=None, memory=None)``, same state
``[S (N,H,E,M), z (N,H,E)]``, same registry entry ``"linear"`` in the recurrent registry.  The
arithmetic of a step -- ``z += K; S += K (x) v; y = (Q . S) / (Q . z + eps)`` (:78-87), five
torch calls in the reference -- is one native launch (``ftb_recurrent_linear_step``); with the
default feature map ``elu(x) + 1`` the map is applied inside the same kernel.

Differences from the reference: CUDA tensors only; the state tensors are fp32 and are always
updated in place (the reference does so when no gradient is recorded, :78-83); recording
gradients through a step is not supported (use the batch form ``CausalLinearAttention`` for
training) and raises.
"""
import ctypes

import torch
from torch.nn import Module

from .... import _native
from ....attention_registry import (Callable, EventDispatcherInstance, Int, Optional,
                                    RecurrentAttentionRegistry)
from ....events import EventDispatcher
from ....feature_maps import elu_feature_map
from ..._utils import check_state


def recurrent_linear_step(Q, K, value, S, z, eps=1e-6, elu_plus_one=False):
    """One native step on features ``Q``, ``K`` (N,H,E) -- or on raw queries / keys when
    ``elu_plus_one`` -- and ``value`` (N,H,M); ``S`` (N,H,E,M) and ``z`` (N,H,E), fp32 and
    contiguous, are updated in place.  Returns the new values (N,H,M)."""
    for t in (Q, K, value, S, z):
        if not t.is_cuda:
            raise RuntimeError("recurrent_linear_step needs CUDA tensors (there is no CPU path)")
    if Q.dtype not in (torch.float32, torch.bfloat16) or K.dtype != Q.dtype or value.dtype != Q.dtype:
        raise RuntimeError("query, key and value must share one dtype, float32 or bfloat16")
    N, H, E = Q.shape
    M = value.shape[2]
    if K.shape != (N, H, E) or value.shape[:2] != (N, H):
        raise RuntimeError("query, key and value shapes do not agree")
    if S.dtype != torch.float32 or z.dtype != torch.float32 or not S.is_contiguous() or not z.is_contiguous():
        raise RuntimeError("the state must be contiguous float32 tensors")
    if S.shape != (N, H, E, M) or z.shape != (N, H, E):
        raise RuntimeError("the state does not match the inputs")
    Q, K, value = (t if t.stride(-1) == 1 or t.shape[-1] <= 1 else t.contiguous() for t in (Q, K, value))
    out = torch.empty(N, H, M, device=Q.device, dtype=Q.dtype)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())   # noqa: E731
    with torch.cuda.device(Q.device):
        st = _native.lib().ftb_recurrent_linear_step(
            ptr(Q), ptr(K), ptr(value), ptr(S), ptr(z), ptr(out), N, H, E, M,
            _native.strides2(Q), _native.strides2(K), _native.strides2(value), _native.strides2(out),
            0 if Q.dtype == torch.float32 else 1,
            _native.FEATURE_ELU1 if elu_plus_one else _native.FEATURE_NONE, float(eps),
            ctypes.c_void_p(torch.cuda.current_stream(Q.device).cuda_stream))
    _native.check(st, "ftb_recurrent_linear_step")
    return out


class RecurrentLinearAttention(Module):
    """``fast_transformers.attention.causal_linear_attention`` as a recurrent model.

    Arguments (as in the reference, ``linear_attention.py:37-45``)
    ---------
        query_dimensions: int, the feature dimension of queries and keys
        feature_map: callable, factory of the feature map (default: elu(x)+1)
        eps: float, added to the denominator (default: 1e-6)
        event_dispatcher: str or EventDispatcher instance
    """

    def __init__(self, query_dimensions, feature_map=None, eps=1e-6, event_dispatcher=""):
        super(RecurrentLinearAttention, self).__init__()
        self.feature_map = (feature_map(query_dimensions) if feature_map
                            else elu_feature_map(query_dimensions))
        self.eps = eps
        self.event_dispatcher = EventDispatcher.get(event_dispatcher)

    def _fused_elu(self):
        f = getattr(self.feature_map, "activation_function", None)
        return getattr(f, "fused_id", None) == "elu+1"

    def forward(self, query, key, value, state=None, memory=None):
        state = check_state(state, memory)
        if state is None:
            self.feature_map.new_feature_map(query.device)
        if torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value)):
            raise RuntimeError("the native recurrent step records no gradients; train with the "
                               "batch form (CausalLinearAttention) or call it under no_grad")
        fused = self._fused_elu()
        if fused:
            Q, K = query, key
        else:
            Q = self.feature_map.forward_queries(query)
            K = self.feature_map.forward_keys(key)
        N, H, D = Q.shape
        M = value.shape[2]
        if state is None:
            Si = torch.zeros(N, H, D, M, device=query.device, dtype=torch.float32)
            Zi = torch.zeros(N, H, D, device=query.device, dtype=torch.float32)
        else:
            Si, Zi = state
        if len(Si) != N:
            raise ValueError("The batch size changed during iteration")
        V = recurrent_linear_step(Q, K, value, Si, Zi, self.eps, elu_plus_one=fused)
        return V, [Si, Zi]

    def _state_of(self, keys, values, key_lengths):
        from ....causal_product import causal_state_sum
        K = self.feature_map.forward_keys(keys)
        if key_lengths is not None:
            K = K * key_lengths.float_matrix[:, :, None, None]
        S = causal_state_sum(K.permute(0, 2, 1, 3), values.permute(0, 2, 1, 3), mode="fp32")
        return [S, K.sum(dim=1).float().contiguous()]

    @torch.no_grad()
    def state_after(self, keys, values, key_lengths=None):
        """The state ``[S, z]`` after a whole prefix processed in batch form: ``keys`` (N,L,H,E)
        and ``values`` (N,L,H,M) as ``CausalLinearAttention`` takes them.  Steps of this module
        continue the sequence from there (prefill in batch form, then decode token by token)."""
        self.feature_map.new_feature_map(keys.device)
        return self._state_of(keys, values, key_lengths)

    @torch.no_grad()
    def prefill(self, queries, keys, values, key_lengths=None):
        """A whole prefix in batch form: ``queries``, ``keys`` (N,L,H,E) and ``values`` (N,L,H,M).
        Returns what ``CausalLinearAttention`` gives for it, (N,L,H,M), and the state ``[S, z]``
        after it, both under ONE draw of a random feature map (``new_feature_map`` is called
        once, as at the first step of a sequence, :64-66 of the reference module)."""
        from ....attention.causal_linear_attention import CausalLinearAttention
        from ....masking import LengthMask, TriangularCausalMask
        N, L = queries.shape[0], queries.shape[1]
        if key_lengths is None:
            key_lengths = LengthMask(queries.new_full((N,), L, dtype=torch.int64))
        self.feature_map.new_feature_map(queries.device)
        same_map = _SameFeatureMap(self.feature_map)
        batch = CausalLinearAttention(queries.shape[3], feature_map=lambda dims: same_map,
                                      eps=self.eps, event_dispatcher=self.event_dispatcher)
        out = batch(queries, keys, values, TriangularCausalMask(L, device=queries.device),
                    key_lengths, key_lengths)
        return out, self._state_of(keys, values, key_lengths)


class _SameFeatureMap(object):
    """An attention's feature map as the batch layer sees it during ``prefill``: the same
    parameters, and no resampling when the layer starts its forward pass."""

    def __init__(self, feature_map):
        self._feature_map = feature_map

    def new_feature_map(self, device):
        return

    def forward_queries(self, x):
        return self._feature_map.forward_queries(x)

    def forward_keys(self, x):
        return self._feature_map.forward_keys(x)

    @property
    def activation_function(self):
        # lets the batch layer recognise the default map and use its native elu(x) + 1 pass
        return getattr(self._feature_map, "activation_function", None)


RecurrentAttentionRegistry.register(
    "linear", RecurrentLinearAttention,
    [
        ("query_dimensions", Int),
        ("feature_map", Optional(Callable)),
        ("event_dispatcher", Optional(EventDispatcherInstance, ""))
    ]
)
# the reference registers the same class under the causal layer's name as well
# (recurrent/attention/self_attention/linear_attention.py:103-110)
RecurrentAttentionRegistry.register(
    "causal-linear", RecurrentLinearAttention,
    [
        ("query_dimensions", Int),
        ("feature_map", Optional(Callable)),
        ("event_dispatcher", Optional(EventDispatcherInstance, ""))
    ]
)
