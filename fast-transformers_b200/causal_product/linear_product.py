"""The NON-causal product ``out_i = Q_i . sum_j K_j^T V_j`` (every position reads the state of
the whole sequence) on the same native library as the causal product.

The reference has no native code for it: ``LinearAttention.forward`` writes it as two
``torch.einsum`` calls (``fast_transformers/attention/linear_attention.py:72-78``).  Here it is the
two phases the causal kernels already consist of, used once each: the whole-range state
(``ftb_causal_state_sum``) and one fixed state applied to every row (``ftb_linear_apply_state``);
the gradients are the same two operations with the roles exchanged:

    S = K^T V            out    = Q S
    R = Q^T G            grad_Q = G S^T      grad_K = V R^T      grad_V = K R
"""
import ctypes

import torch

from .. import _native
from ..settings import get_mode
from . import _check_cuda, _dtype_id, _like, _mode_id, _ptr, _rowmajor, causal_state_sum


def linear_apply_state(a, state, out=None, mode=None, transposed=False):
    """``out[n,h,l,:] = a[n,h,l,:] . state[n,h]`` for (N, H, L, Da) ``a`` and a float32 state of
    shape (N, H, Da, Dc) -- or (N, H, Dc, Da), applied as its transpose, when ``transposed``."""
    dev = _check_cuda(a)
    dt = _dtype_id(a)
    N, H, L, Da = a.shape
    if state.dtype != torch.float32 or state.dim() != 4 or state.device != dev or \
            state.shape[:2] != (N, H) or state.shape[3 if transposed else 2] != Da:
        raise RuntimeError("state must be a float32 (N, H, %s) tensor on the inputs' device"
                           % ("Dc, Da" if transposed else "Da, Dc"))
    Dc = state.shape[2 if transposed else 3]
    state = state.contiguous()
    a = _rowmajor(a)
    if out is None:
        out = torch.empty((N, H, L, Dc), device=dev, dtype=a.dtype)
    elif out.shape != (N, H, L, Dc) or out.dtype != a.dtype or (Dc > 1 and out.stride(3) != 1):
        raise RuntimeError("out must be a row-contiguous (N, H, L, Dc) tensor of the input dtype")
    with torch.cuda.device(dev):
        st = _native.lib().ftb_linear_apply_state(
            _ptr(a), _ptr(state), _ptr(out), N, H, L, Da, Dc, _native.strides3(a),
            _native.strides3(out), dt, _mode_id(mode), int(bool(transposed)),
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _native.check(st, "ftb_linear_apply_state")
    return out


class LinearDotProduct(torch.autograd.Function):
    """``out = Q (K^T V)`` for (N, H, L, D) queries, (N, H, S, D) keys and (N, H, S, M) values;
    saves Q, K, V and the (N, H, D, M) state."""

    @staticmethod
    def forward(ctx, Q, K, V):
        _check_cuda(Q, K, V)
        if K.shape[:3] != V.shape[:3] or Q.shape[:2] != K.shape[:2] or Q.shape[3] != K.shape[3]:
            raise RuntimeError("shape mismatch between queries, keys and values")
        if not (Q.dtype == K.dtype == V.dtype):
            raise RuntimeError("queries, keys and values must share one dtype")
        ctx.mode = get_mode()
        S = causal_state_sum(K.data, V.data, mode=ctx.mode)
        M = V.shape[3]
        # the result in the memory order of Q (see CausalDotProduct.forward)
        out = _like(Q) if Q.shape[3] == M else None
        out = linear_apply_state(Q.data, S, out, ctx.mode)
        ctx.save_for_backward(Q, K, V, S)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V, S = ctx.saved_tensors
        G = grad_out if grad_out.dtype == Q.dtype else grad_out.to(Q.dtype)
        need = ctx.needs_input_grad
        gQ = gK = gV = None
        if need[0]:
            gQ = linear_apply_state(G, S, _like(Q), ctx.mode, transposed=True)
        if need[1] or need[2]:
            R = causal_state_sum(Q.data, G, mode=ctx.mode)
            if need[1]:
                gK = linear_apply_state(V.data, R, _like(K), ctx.mode, transposed=True)
            if need[2]:
                gV = linear_apply_state(K.data, R, _like(V), ctx.mode)
        return gQ, gK, gV


linear_dot_product = LinearDotProduct.apply
