"""Causally masked linear attention, O(L D M) per head.

Mirror of ``fast_transformers/attention/causal_linear_attention.py``: ``causal_linear``
(:19-24), ``CausalLinearAttention`` (:27-104) and its ``"causal-linear"`` registry entry
with the same parameter tuple (:109-116).

    Q = phi(queries); K = phi(keys) * key_length_mask
    Z_i = 1 / (Q_i . sum_{j<=i} K_j + eps)
    out_i = Z_i * Q_i . sum_{j<=i} K_j^T V_j

What differs from the reference is data movement only: the kernels take (N, L, H, dim)
storage through strides and write their results in that order, so the four
permute+contiguous copies of ``causal_linear`` are views here; the default feature map and
the key-length mask are one native pass; and the normaliser comes out of the same kernel
launch as the product in ``"fp32"`` mode (V is extended by a column of ones, whose output
column is Q_i . cumsum(K)_i) or out of streaming kernels of its own in ``"mma"`` mode.
"""
import torch
from torch.nn import Module

from ..attention_registry import (AttentionRegistry, Callable, EventDispatcherInstance, Int,
                                  Optional)
from ..causal_product import (causal_dot_backward_cuda, causal_dot_product, causal_dot_product_cuda,
                              causal_normaliser_backward_elu_raw,
                              causal_normaliser, causal_normaliser_backward_raw,
                              causal_normaliser_raw)
from ..events import EventDispatcher
from ..feature_maps import (elu_feature_map, elu_plus_one_backward_raw, elu_plus_one_forward_raw,
                            elu_plus_one_native, is_default_elu_map)
from ..settings import get_mode


def causal_linear(Q, K, V):
    """(N, L, H, dim) in, (N, L, H, M) out.  The permutes are views: the kernels read and
    write the (N, L, H, dim) storage directly through strides."""
    out = causal_dot_product(Q.permute(0, 2, 1, 3), K.permute(0, 2, 1, 3), V.permute(0, 2, 1, 3))
    return out.permute(0, 2, 1, 3)


# The one-node form of the layer body (below) is used whenever it applies; tests switch it off to
# compare it with the chain of separate autograd nodes.
fused_node_enabled = True


def _division_backward(gy, y, den, eps):
    """``grad_out = grad_y * Z`` and ``grad_den = -Z * sum_m grad_y * y`` for ``Z = 1 / (den + eps)``;
    ``gy``, ``y`` (N, L, H, M), ``den`` the (N, H, L) view of (N, L, H) storage.  One native pass for
    contiguous fp32 rows of 16, 32, 64 or 128 values, the torch formulation otherwise."""
    N, L, H, M = y.shape
    den_nlh = den.permute(0, 2, 1)
    if (y.dtype == torch.float32 and den.dtype == torch.float32 and M in (16, 32, 64, 128)
            and y.is_contiguous() and den_nlh.is_contiguous() and y.numel() > 0):
        import ctypes
        from .. import _native
        gy = gy.contiguous()
        grad_out = torch.empty_like(y)
        grad_den = torch.empty((N, L, H), device=y.device, dtype=torch.float32)
        vp = ctypes.c_void_p
        with torch.cuda.device(y.device):
            st = _native.lib().ftb_normalised_output_grads(
                vp(gy.data_ptr()), vp(y.data_ptr()), vp(den_nlh.data_ptr()), vp(grad_out.data_ptr()),
                vp(grad_den.data_ptr()), N * L * H, M, float(eps),
                vp(torch.cuda.current_stream(y.device).cuda_stream))
        _native.check(st, "ftb_normalised_output_grads")
        return grad_out, grad_den
    Z = 1 / (den_nlh + eps)
    return gy * Z[..., None], -(Z * (gy * y).sum(-1))


class _FusedElu1CausalLinear(torch.autograd.Function):
    """The whole layer body for the default feature map as ONE autograd node:

        Q = elu(q) + 1;  K = (elu(k) + 1) * key_mask;  den_l = Q_l . sum_{j<=l} K_j
        y_l = (Q_l . sum_{j<=l} K_j^T V_j) / (den_l + eps)

    (``causal_linear_attention.py:75-104``) on (N, L, H, .) tensors with L = S.  Built from the
    same native passes as the unfused path; what changes is what is kept for the backward: the
    raw queries and keys, V, the (N, H, L) denominator and the result -- not the feature tensors
    Q and K (each as large as the input, otherwise saved twice: by the feature map and by the
    product) nor the unnormalised product.  The backward recomputes Q and K (one native pass
    each).  With y = out * Z, Z = 1 / (den + eps):

        grad_out = grad_y * Z            grad_den = -Z * sum_m grad_y * y
    """

    @staticmethod
    def forward(ctx, queries, keys, values, key_mask, eps, mode):
        xq, xk = queries.contiguous(), keys.contiguous()
        w = None if key_mask is None else key_mask.to(torch.float32).contiguous()
        Q = elu_plus_one_forward_raw(xq, None)
        K = elu_plus_one_forward_raw(xk, w)
        Qp, Kp, Vp = Q.permute(0, 2, 1, 3), K.permute(0, 2, 1, 3), values.permute(0, 2, 1, 3)
        den = causal_normaliser_raw(Qp, Kp)                          # (N, H, L) view of (N, L, H)
        N, L, H, M = values.shape
        y = torch.empty((N, L, H, M), device=values.device, dtype=values.dtype)
        kept = []
        if mode == "mma" and den.dtype == torch.float32 and Q.shape[3] == M == 64:
            # 1 / (den + eps) is applied by the scan as it stores its rows
            causal_dot_product_cuda(Qp, Kp, Vp, y.permute(0, 2, 1, 3), mode, keep_workspace=kept,
                                    row_den=den, eps=eps)
        else:
            causal_dot_product_cuda(Qp, Kp, Vp, y.permute(0, 2, 1, 3), mode, keep_workspace=kept)
            Z = 1 / (den.permute(0, 2, 1) + eps)                     # (N, L, H)
            y.mul_(Z[..., None])
        ctx.save_for_backward(xq, xk, values, w, den, y)
        ctx.eps, ctx.mode = eps, mode
        ctx.forward_workspace = kept[0] if kept else None
        return y

    @staticmethod
    def backward(ctx, grad_y):
        xq, xk, values, w, den, y = ctx.saved_tensors
        Q = elu_plus_one_forward_raw(xq, None)
        K = elu_plus_one_forward_raw(xk, w)
        Qp, Kp, Vp = Q.permute(0, 2, 1, 3), K.permute(0, 2, 1, 3), values.permute(0, 2, 1, 3)
        gy = grad_y if grad_y.dtype == y.dtype else grad_y.to(y.dtype)
        grad_out, grad_den = _division_backward(gy, y, den, ctx.eps)   # (N, L, H, M), (N, L, H)
        gQ, gK, gV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(values)
        causal_dot_backward_cuda(Qp, Kp, Vp, grad_out.permute(0, 2, 1, 3), gQ.permute(0, 2, 1, 3),
                                 gK.permute(0, 2, 1, 3), gV.permute(0, 2, 1, 3), ctx.mode,
                                 forward_workspace=ctx.forward_workspace)
        # the denominator's gradients join the product's in place, and the sum goes through the
        # feature map's derivative on its way back to memory
        if causal_normaliser_backward_elu_raw(Qp, Kp, grad_den.permute(0, 2, 1), gQ.permute(0, 2, 1, 3),
                                              gK.permute(0, 2, 1, 3), xq.permute(0, 2, 1, 3),
                                              xk.permute(0, 2, 1, 3), w):
            return gQ, gK, gV, None, None, None
        causal_normaliser_backward_raw(Qp, Kp, grad_den.permute(0, 2, 1),
                                       add_to=(gQ.permute(0, 2, 1, 3), gK.permute(0, 2, 1, 3)))
        return (elu_plus_one_backward_raw(xq, gQ, None), elu_plus_one_backward_raw(xk, gK, w), gV,
                None, None, None)


class CausalLinearAttention(Module):
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

    def _make_sizes_compatible(self, Q, K):
        """Slice K to L rows, or pad it with zero rows, when L != S (:57-69)."""
        N, L, H, E = Q.shape
        S = K.shape[1]
        if L == S:
            return Q, K
        if L < S:
            return Q, K[:, :L, :, :]
        return Q, torch.cat([K, K.new_zeros(N, L - S, H, E)], dim=1)

    def forward(self, queries, keys, values, attn_mask, query_lengths, key_lengths):
        self.feature_map.new_feature_map(queries.device)
        if not attn_mask.lower_triangular:
            raise RuntimeError("CausalLinearAttention only supports full lower triangular masks")
        native_map = (is_default_elu_map(self.feature_map) and queries.is_cuda
                      and queries.dtype in (torch.float32, torch.bfloat16))
        mode = get_mode()
        if (fused_node_enabled and native_map and queries.shape[1] == keys.shape[1] == values.shape[1]
                and keys.dtype == queries.dtype and values.dtype == queries.dtype
                and queries.shape[3] in (16, 32, 64, 128)
                and (mode == "mma" or values.shape[3] % 64 == 0)
                and tuple(key_lengths.float_matrix.shape) == tuple(keys.shape[:2])):
            # the common case (L = S, a width the streaming denominator kernels take): the whole
            # body as one autograd node that keeps the raw inputs instead of the feature tensors
            return _FusedElu1CausalLinear.apply(queries, keys, values, key_lengths.float_matrix,
                                                self.eps, mode)
        if native_map:
            # elu(x) + 1 and the key-length mask in one native pass each (and one each backward)
            Q = elu_plus_one_native(queries)
            K = elu_plus_one_native(keys, key_lengths.float_matrix)
        else:
            Q = self.feature_map.forward_queries(queries)
            K = self.feature_map.forward_keys(keys)
            K = K * key_lengths.float_matrix[:, :, None, None]
        Q, K = self._make_sizes_compatible(Q, K)

        # Bring V to L rows as well.  The reference leaves V as it is (for L > S its kernel
        # then reads past the S rows of V, multiplied by zero keys); explicit rows give the
        # same result without touching memory that is not V's.
        N, L, H, _ = Q.shape
        S = values.shape[1]
        if S > L:
            values = values[:, :L]
        elif S < L:
            values = torch.cat([values, values.new_zeros(N, L - S, H, values.shape[3])], dim=1)

        M = values.shape[3]
        E = Q.shape[3]
        fp32_mode = get_mode() == "fp32"
        if fp32_mode and (M % 64 != 0 or E > 256):
            # One extra value column of ones: its output column is Q_i . sum_{j<=i} K_j, the
            # denominator, so product and normaliser share one pass over Q and K.  (Free while
            # M + 1 columns still fit the kernel's 64-column tile; at M = 64 it would cost a
            # second tile, i.e. the whole product again.)
            Vx = torch.cat([values, values.new_ones(N, L, H, 1)], dim=-1)
            out = causal_linear(Q, K, Vx)
            Z = 1 / (out[..., M] + self.eps)
            return (out[..., :M] * Z[..., None]).contiguous()
        if E > 256:
            # wider than the denominator kernels take: the reference's formulation (:95)
            Z = 1 / (torch.einsum("nlhi,nlhi->nlh", Q, K.cumsum(1)) + self.eps)
            return (causal_linear(Q, K, values) * Z[:, :, :, None]).contiguous()
        # The denominator Q_i . sum_{j<=i} K_j from streaming kernels of its own (and so its
        # gradients): the tensor-core kernels take D = M only, so the column of ones cannot
        # ride along there.  The reference's way (:95) -- a cumulative sum of K and a row-wise
        # dot product as torch calls, plus their autograd -- took half of an encoder step here
        # (12 ms of 24 ms per layer at N16 L8192 H8 E64).
        den = causal_normaliser(Q.permute(0, 2, 1, 3), K.permute(0, 2, 1, 3))      # (N, H, L)
        Z = 1 / (den.permute(0, 2, 1) + self.eps)
        return (causal_linear(Q, K, values) * Z[:, :, :, None]).contiguous()


AttentionRegistry.register(
    "causal-linear", CausalLinearAttention,
    [
        ("query_dimensions", Int),
        ("feature_map", Optional(Callable)),
        ("event_dispatcher", Optional(EventDispatcherInstance, ""))
    ]
)
