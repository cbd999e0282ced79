"""Causal dot product ``V'_i = Q_i . sum_{j<=i} K_j^T V_j`` on B200.

Mirror of ``fast_transformers/causal_product/__init__.py``: the same autograd Function
(``CausalDotProduct`` with class-level per-device tables ``dot`` / ``dot_backward``, :20-30),
the same alias ``causal_dot_product = CausalDotProduct.apply`` (:78) and native functions
with the reference's in-place signatures (``causal_product_cuda.cu:1471-1483``):

    causal_dot_product_cuda(queries, keys, values, product) -> None
    causal_dot_backward_cuda(queries, keys, values, grad_out, grad_q, grad_k, grad_v) -> None

Differences, all deliberate: there is no CPU entry (``dot["cpu"]`` is None and CPU tensors
raise -- this package has no CPU path); kernels run on torch's current stream instead of
the legacy default stream; outputs need not be zero on entry; bf16 tensors are accepted in
addition to fp32 (bf16 in, bf16 out, fp32 state).  In ``"mma"`` mode fp32 tensors may have any
query / value widths that are multiples of 64 (the Favor map gives D = 256; 128-wide heads): the
library takes the sums over 64-wide feature blocks inside the tensor cores.  The mode
``"tf32x3"`` names the accuracy tier of ``"fp32"`` on the tensor cores (split operands; fp32 tensors
with D = M = 64, everything else runs as ``"fp32"``).
"""
import ctypes

import torch

from .. import _native
from ..settings import get_mode

_DTYPES = {torch.float32: _native.F32, torch.bfloat16: _native.BF16}


def _dtype_id(t):
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        # the reference raises the same kind of error from accessor<float>
        raise RuntimeError("expected scalar type Float (or BFloat16) but found %s" % t.dtype)


def _check_cuda(*ts):
    dev = ts[0].device
    for t in ts:
        if t.device.type != "cuda":
            raise RuntimeError(
                "fast_transformers_b200 runs on CUDA (sm_100a) only; got a %s tensor. "
                "There is no CPU implementation." % t.device.type)
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
        if t.dim() != 4:
            raise RuntimeError("expected 4-dimensional (N, H, L, dim) tensors")
    return dev


def _rowmajor(t):
    """The kernels need a contiguous last dimension (the reference asserts stride(3)==1)."""
    return t if (t.shape[3] <= 1 or t.stride(3) == 1) else t.contiguous()


def _like(t):
    """An uninitialised buffer of ``t``'s shape that the kernels can write: in the memory order
    of ``t`` when its rows are contiguous (the layer's (N, L, H, dim) storage viewed as
    (N, H, L, dim) keeps its order, and the caller's permute back is then a view), row-major
    otherwise (a transposed input, say)."""
    if t.shape[3] <= 1 or t.stride(3) == 1:
        return torch.empty_like(t)
    return torch.empty(t.shape, dtype=t.dtype, device=t.device)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _workspace(nbytes, device):
    if nbytes == 0:
        return None, 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return ws, nbytes


def _mode_id(mode, split_ok=False):
    """Native id of ``mode`` (default: the thread's setting).  ``"tf32x3"`` names an accuracy tier:
    the split-operand tensor-core kernels where the caller says they apply (``split_ok``: the
    causal product or its backward, fp32, D = M = 64, no states), the fp32 kernels elsewhere."""
    name = mode or get_mode()
    if name == "tf32x3" and not split_ok:
        name = "fp32"
    return _native.MODE_IDS[name]


def _split_ok(t, D, M, *states):
    return t.dtype == torch.float32 and D == 64 and M == 64 and all(s is None or s is False for s in states)


def _state_ok(s, N, H, D, M, dev, name):
    if s is None:
        return None
    if s.dtype != torch.float32 or s.shape != (N, H, D, M) or s.device != dev:
        raise RuntimeError("%s must be a float32 (N, H, D, M) tensor on the inputs' device" % name)
    return s.contiguous()


def workspace_bytes(N, H, L, D, M, dtype, mode=None, backward=False, want_state=False):
    """Scratch bytes of one forward (or backward) call; see ``ftb_causal_workspace_bytes``."""
    split = dtype == torch.float32 and D == 64 and M == 64 and not want_state
    return _native.lib().ftb_causal_workspace_bytes(
        N, H, L, D, M, _DTYPES[dtype], _mode_id(mode, split), int(backward), int(want_state))


def causal_dot_product_cuda(queries, keys, values, product, mode=None, initial_state=None,
                            final_state=None, keep_workspace=None, workspace=None,
                            workspace_has_states=False, row_den=None, eps=0.0):
    """Fill ``product`` (N, H, L, M) in place -- the reference's native forward signature
    (``causal_product_cuda.cu:1273-1276``), plus optional fp32 states (N, H, D, M).  With
    ``row_den`` (fp32, (N, H, L), any strides) row i of the result is divided by
    ``row_den[n, h, i] + eps`` as it is stored (``ftb_causal_dot_product_normalised``; ``"mma"``
    mode, no states)."""
    dev = _check_cuda(queries, keys, values, product)
    dt = _dtype_id(queries)
    for t in (keys, values, product):
        if t.dtype != queries.dtype:
            raise RuntimeError("expected scalar type %s but found %s" % (queries.dtype, t.dtype))
    N, H, L, D = queries.shape
    M = values.shape[3]
    if values.shape[:2] == (N, H) and values.shape[2] > L:
        # The reference's layer hands over V with all S rows when L < S
        # (causal_linear_attention.py:98-102); its kernels walk the L rows of Q and never look
        # at the rest (tests/attention/test_causal_linear_attention.py:33-39).  Same here.
        values = values[:, :, :L]
    if keys.shape != (N, H, L, D) or values.shape[:3] != (N, H, L) or \
            product.shape != (N, H, L, M):
        raise RuntimeError("shape mismatch between queries, keys, values and product")
    if product.shape[3] > 1 and product.stride(3) != 1:
        raise RuntimeError("product must have a contiguous last dimension")
    q, k, v = _rowmajor(queries), _rowmajor(keys), _rowmajor(values)
    initial_state = _state_ok(initial_state, N, H, D, M, dev, "initial_state")
    if final_state is not None and (final_state.dtype != torch.float32 or
                                    final_state.shape != (N, H, D, M) or
                                    not final_state.is_contiguous()):
        raise RuntimeError("final_state must be a contiguous float32 (N, H, D, M) tensor")
    L_ = _native.lib()
    m = _mode_id(mode, _split_ok(queries, D, M, initial_state, final_state, workspace_has_states))
    if (mode or get_mode()) == "tf32x3" and m != _native.MODE_MMA_X3:
        keep_workspace = None      # fp32-kernel states: not what a split-operand backward reads
    with torch.cuda.device(dev):
        nbytes = L_.ftb_causal_workspace_bytes(N, H, L, D, M, dt, m, 0, int(final_state is not None))
        if workspace is not None:
            if workspace.numel() * workspace.element_size() < nbytes:
                raise RuntimeError("workspace tensor is too small")
            ws, nbytes = workspace, workspace.numel() * workspace.element_size()
        else:
            ws, nbytes = _workspace(nbytes, dev)
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        if row_den is not None:
            if initial_state is not None or final_state is not None or workspace_has_states:
                raise RuntimeError("the normalised product takes no states")
            if row_den.dtype != torch.float32 or row_den.shape != (N, H, L) or row_den.device != dev:
                raise RuntimeError("row_den must be a float32 (N, H, L) tensor on the inputs' device")
            dstr = (ctypes.c_int64 * 3)(*row_den.stride())
            st = L_.ftb_causal_dot_product_normalised(
                _ptr(q), _ptr(k), _ptr(v), _ptr(row_den), _ptr(product), N, H, L, D, M,
                _native.strides3(q), _native.strides3(k), _native.strides3(v), dstr,
                _native.strides3(product), dt, m, float(eps), _ptr(ws), nbytes, stream)
        else:
            st = L_.ftb_causal_dot_product(
                _ptr(q), _ptr(k), _ptr(v), _ptr(product), N, H, L, D, M,
                _native.strides3(q), _native.strides3(k), _native.strides3(v),
                _native.strides3(product), dt, m, _ptr(initial_state), _ptr(final_state),
                int(bool(workspace_has_states)), _ptr(ws), nbytes, stream)
    _native.check(st, "ftb_causal_dot_product")
    if keep_workspace is not None:
        # the per-segment forward states; the backward pass reuses them if handed back
        keep_workspace.append(ws)


def causal_dot_backward_cuda(queries, keys, values, grad_out, grad_queries, grad_keys,
                             grad_values, mode=None, initial_state=None,
                             initial_grad_state=None, forward_workspace=None, workspace=None,
                             workspace_has_grad_states=False):
    """Fill the three gradients in place -- the reference's native backward signature
    (``causal_product_cuda.cu:1438-1444``).  ``grad_out`` may be any view (expanded,
    permuted); it is made row-contiguous only if its last stride is not 1.  A gradient buffer
    given as ``None`` is not computed (the sequence-parallel path asks for grad_Q first and
    for grad_K, grad_V once the reverse states have arrived)."""
    wanted = [t for t in (grad_queries, grad_keys, grad_values) if t is not None]
    if not wanted:
        raise RuntimeError("no gradient was asked for")
    dev = _check_cuda(queries, keys, values, grad_out, *wanted)
    dt = _dtype_id(queries)
    N, H, L, D = queries.shape
    M = values.shape[3]
    if values.shape[:2] == (N, H) and values.shape[2] > L:
        # V longer than the queries (see the forward): rows past L take no part, their gradient
        # is zero (the reference relies on its zero-initialised buffer for that)
        values = values[:, :, :L]
        if grad_values is not None and grad_values.shape[2] > L:
            grad_values[:, :, L:].zero_()
            grad_values = grad_values[:, :, :L]
            wanted = [t for t in (grad_queries, grad_keys, grad_values) if t is not None]
    if grad_out.dtype != queries.dtype:
        grad_out = grad_out.to(queries.dtype)
    if grad_out.shape != (N, H, L, M):
        raise RuntimeError("grad_out has the wrong shape")
    q, k, v, g = (_rowmajor(t) for t in (queries, keys, values, grad_out))
    for t in wanted:
        if t.dtype != queries.dtype or (t.shape[3] > 1 and t.stride(3) != 1):
            raise RuntimeError("gradient buffers must match the input dtype and be row-contiguous")
    initial_state = _state_ok(initial_state, N, H, D, M, dev, "initial_state")
    initial_grad_state = _state_ok(initial_grad_state, N, H, D, M, dev, "initial_grad_state")
    L_ = _native.lib()
    m = _mode_id(mode, _split_ok(queries, D, M, initial_state, initial_grad_state, workspace_has_grad_states))
    with torch.cuda.device(dev):
        nbytes = L_.ftb_causal_workspace_bytes(N, H, L, D, M, dt, m, 1, 0)
        if workspace is not None:
            if workspace.numel() * workspace.element_size() < nbytes:
                raise RuntimeError("workspace tensor is too small")
            ws, nbytes = workspace, workspace.numel() * workspace.element_size()
        else:
            ws, nbytes = _workspace(nbytes, dev)
        st = L_.ftb_causal_dot_backward(
            _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(grad_queries), _ptr(grad_keys),
            _ptr(grad_values), N, H, L, D, M,
            _native.strides3(q), _native.strides3(k), _native.strides3(v), _native.strides3(g),
            _native.strides3(grad_queries if grad_queries is not None else q),
            _native.strides3(grad_keys if grad_keys is not None else k),
            _native.strides3(grad_values if grad_values is not None else v), dt, m, _ptr(initial_state),
            _ptr(initial_grad_state), _ptr(forward_workspace),
            int(bool(workspace_has_grad_states)), _ptr(ws), nbytes,
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _native.check(st, "ftb_causal_dot_backward")


def causal_state_sum(x, y, mode=None, workspace=None, reverse=False):
    """``sum_l x[n,h,l,:] (x) y[n,h,l,:]`` as a float32 (N, H, D, M) tensor: the state a
    range of positions contributes to the ranges after it (x=K, y=V) or before it
    (x=Q, y=grad_out)."""
    dev = _check_cuda(x, y)
    dt = _dtype_id(x)
    if y.dtype != x.dtype:
        raise RuntimeError("expected scalar type %s but found %s" % (x.dtype, y.dtype))
    N, H, L, D = x.shape
    M = y.shape[3]
    x, y = _rowmajor(x), _rowmajor(y)
    state = torch.empty(N, H, D, M, dtype=torch.float32, device=dev)
    L_ = _native.lib()
    m = _mode_id(mode)
    with torch.cuda.device(dev):
        nbytes = L_.ftb_causal_workspace_bytes(N, H, L, D, M, dt, m, 0, 1)
        if workspace is not None:
            # a caller-kept workspace: the per-segment states left in it can be handed to the
            # forward (workspace_has_states) or backward (workspace_has_grad_states) call
            if workspace.numel() * workspace.element_size() < nbytes:
                raise RuntimeError("workspace tensor is too small")
            ws, nbytes = workspace, workspace.numel() * workspace.element_size()
        else:
            ws, nbytes = _workspace(nbytes, dev)
        st = L_.ftb_causal_state_sum(
            _ptr(x), _ptr(y), _ptr(state), N, H, L, D, M, _native.strides3(x),
            _native.strides3(y), dt, m, int(bool(reverse)), _ptr(ws), nbytes,
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _native.check(st, "ftb_causal_state_sum")
    return state


def causal_state_parts(x, y, workspace, mode=None):
    """Partial sums of ``sum_l x_l (x) y_l`` left in ``workspace`` (a uint8 tensor of at least
    ``workspace_bytes(..., want_state=True)`` bytes): returns the number of (D, M) float32 blocks per
    (batch, head) pair that add up to the pair's state, or 0 when this shape and mode keep no raw
    partial sums (nothing is launched then).  The workspace can be handed to the forward / backward
    call like the one ``causal_state_sum`` fills."""
    dev = _check_cuda(x, y)
    dt = _dtype_id(x)
    N, H, L, D = x.shape
    M = y.shape[3]
    L_ = _native.lib()
    m = _mode_id(mode)
    parts = L_.ftb_causal_state_parts(N, H, L, D, M, dt, m)
    if parts == 0:
        return 0
    x, y = _rowmajor(x), _rowmajor(y)
    with torch.cuda.device(dev):
        st = L_.ftb_causal_state_sum(
            _ptr(x), _ptr(y), None, N, H, L, D, M, _native.strides3(x), _native.strides3(y), dt, m, 0,
            _ptr(workspace), workspace.numel() * workspace.element_size(),
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _native.check(st, "ftb_causal_state_sum")
    return parts


def _no_cpu(*args, **kwargs):
    raise RuntimeError("fast_transformers_b200 has no CPU implementation of causal_dot_product; "
                       "move the tensors to a CUDA (B200) device")


class CausalDotProduct(torch.autograd.Function):
    """Compute the weighted sum of values but attending only to previous values.

    Same contract as ``fast_transformers.causal_product.CausalDotProduct`` (:20-74): saves
    only Q, K, V; allocates the outputs here and lets the native function fill them."""
    dot = {"cpu": _no_cpu, "cuda": causal_dot_product_cuda}
    dot_backward = {"cpu": _no_cpu, "cuda": causal_dot_backward_cuda}

    @staticmethod
    def forward(ctx, Q, K, V):
        ctx.save_for_backward(Q, K, V)
        ctx.mode = get_mode()
        N, H, L, _ = Q.shape
        M = V.shape[3]
        # the reference allocates zeros (its fallback kernels accumulate); ours overwrite.  The
        # result takes the memory order of V (the layer passes (N, L, H, M) storage viewed as
        # (N, H, L, M)): the kernels write through strides, and the caller's permute back is
        # then contiguous instead of a copy
        product = _like(V) if V.shape == (N, H, L, M) else \
            torch.empty((N, H, L, M), device=Q.device, dtype=Q.dtype)
        kept = []
        fwd = CausalDotProduct.dot[Q.device.type]
        if fwd is causal_dot_product_cuda:
            fwd(Q.data, K.data, V.data, product, ctx.mode, keep_workspace=kept)
        else:   # a replacement installed with the reference's four-argument signature
            fwd(Q.data, K.data, V.data, product)
        ctx.forward_workspace = kept[0] if kept else None
        return product

    @staticmethod
    def backward(ctx, grad_out):
        Q, K, V = ctx.saved_tensors
        bwd = CausalDotProduct.dot_backward[Q.device.type]
        native = bwd is causal_dot_backward_cuda
        # the native function skips a gradient whose buffer is None (a constant V, for example
        # the column of ones behind the layer's normaliser, costs no grad_V scan)
        need = list(ctx.needs_input_grad[:3])
        if not native or not any(need):
            need = [True, True, True]
        # gradients in the memory order of their inputs (see forward)
        grad_Q = _like(Q) if need[0] else None
        grad_K = _like(K) if need[1] else None
        grad_V = _like(V) if need[2] else None
        if native:
            bwd(Q.data, K.data, V.data, grad_out, grad_Q, grad_K, grad_V, ctx.mode,
                forward_workspace=ctx.forward_workspace)
        else:
            bwd(Q.data, K.data, V.data, grad_out, grad_Q, grad_K, grad_V)
        return grad_Q, grad_K, grad_V


# Alias the autograd functions to python style snake case naming
causal_dot_product = CausalDotProduct.apply


def _strides_nhl(t):
    s = t.stride()
    return (ctypes.c_int64 * 3)(s[0], s[1], s[2])


def causal_normaliser_raw(Q, K):
    """``den[n,h,l] = Q[n,h,l] . sum_{j<=l} K[n,h,j]`` for (N, H, L, D) views, no autograd; the
    result has the memory order of ``Q[..., 0]``."""
    dev = _check_cuda(Q, K)
    if Q.shape != K.shape or Q.dtype != K.dtype:
        raise RuntimeError("Q and K must have one shape and dtype")
    dt = _dtype_id(Q)
    N, H, L, D = Q.shape
    q, k = _rowmajor(Q), _rowmajor(K)
    den = torch.empty_like(Q[..., 0]) if D > 0 else torch.empty((N, H, L), device=dev, dtype=Q.dtype)
    L_ = _native.lib()
    with torch.cuda.device(dev):
        nbytes = L_.ftb_causal_normaliser_workspace_bytes(N, H, L, D, 0)
        ws, nbytes = _workspace(nbytes, dev)
        st = L_.ftb_causal_normaliser(
            _ptr(q), _ptr(k), _ptr(den), N, H, L, D, _native.strides3(q), _native.strides3(k),
            _strides_nhl(den), dt, _ptr(ws), nbytes,
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _native.check(st, "ftb_causal_normaliser")
    return den


def causal_normaliser_backward_raw(Q, K, grad_den, need_q=True, need_k=True, add_to=None):
    """Gradients of ``causal_normaliser_raw``: ``gQ_l = g_l * sum_{j<=l} K_j``,
    ``gK_j = sum_{l>=j} g_l * Q_l`` (either may be skipped), in the memory order of Q and K.
    ``add_to=(gQ, gK)``: the gradients are ADDED to these tensors (row-contiguous, of Q's and K's
    shape and dtype; ``None`` skips one) instead of returned in new ones."""
    dev = Q.device
    dt = _dtype_id(Q)
    N, H, L, D = Q.shape
    q, k = _rowmajor(Q), _rowmajor(K)
    g = grad_den if grad_den.dtype == Q.dtype else grad_den.to(Q.dtype)
    if add_to is not None:
        gq, gk = add_to
        for t, like in ((gq, Q), (gk, K)):
            if t is not None and (t.shape != like.shape or t.dtype != like.dtype or t.stride(3) != 1):
                raise RuntimeError("add_to tensors must match Q / K in shape and dtype and be row-contiguous")
    else:
        gq = _like(Q) if need_q else None
        gk = _like(K) if need_k else None
    if gq is None and gk is None:
        return None, None
    L_ = _native.lib()
    fn = L_.ftb_causal_normaliser_backward_add if add_to is not None else L_.ftb_causal_normaliser_backward
    with torch.cuda.device(dev):
        nbytes = L_.ftb_causal_normaliser_workspace_bytes(N, H, L, D, 1)
        ws, nbytes = _workspace(nbytes, dev)
        st = fn(
            _ptr(q), _ptr(k), _ptr(g), _ptr(gq), _ptr(gk), N, H, L, D, _native.strides3(q),
            _native.strides3(k), _strides_nhl(g), _native.strides3(gq if gq is not None else q),
            _native.strides3(gk if gk is not None else k), dt, _ptr(ws), nbytes,
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _native.check(st, "ftb_causal_normaliser_backward")
    return gq, gk


def causal_normaliser_backward_elu_raw(Q, K, grad_den, grad_q, grad_k, xq, xk, key_weights=None):
    """In place: ``grad_q <- (grad_q + n_q) phi'(xq)``, ``grad_k <- (grad_k + n_k) w phi'(xk)`` with
    ``n_q``, ``n_k`` the denominator's gradients (``causal_normaliser_backward_raw``),
    ``phi(x) = elu(x) + 1`` and ``w`` the (N, L) key weights -- the tail of the layer's backward in two
    launches (``ftb_causal_normaliser_backward_elu``).  All tensors (N, H, L, D) views with a
    contiguous last dimension; returns False, with nothing changed, for shapes the kernels do not
    take."""
    dev = Q.device
    dt = _dtype_id(Q)
    N, H, L, D = Q.shape
    ok = D in (16, 32, 64, 128)
    for t in (Q, K, grad_q, grad_k, xq, xk):
        ok = ok and t.shape == Q.shape and t.dtype == Q.dtype and t.stride(3) == 1 and \
            all(s % 4 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0
    if not ok:
        return False
    g = grad_den if grad_den.dtype == Q.dtype else grad_den.to(Q.dtype)
    w = None if key_weights is None else key_weights.to(torch.float32).contiguous()
    L_ = _native.lib()
    with torch.cuda.device(dev):
        nbytes = L_.ftb_causal_normaliser_workspace_bytes(N, H, L, D, 1)
        ws, nbytes = _workspace(nbytes, dev)
        st = L_.ftb_causal_normaliser_backward_elu(
            _ptr(Q), _ptr(K), _ptr(g), _ptr(grad_q), _ptr(grad_k), _ptr(xq), _ptr(xk), _ptr(w), N, H, L, D,
            _native.strides3(Q), _native.strides3(K), _strides_nhl(g), _native.strides3(grad_q),
            _native.strides3(grad_k), _native.strides3(xq), _native.strides3(xk), dt, _ptr(ws), nbytes,
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _native.check(st, "ftb_causal_normaliser_backward_elu")
    return True


class CausalNormaliser(torch.autograd.Function):
    """``den[n,h,l] = Q[n,h,l] . sum_{j<=l} K[n,h,j]`` for (N, H, L, D) views: the denominator of
    the attention layer, which the reference computes as
    ``torch.einsum("nlhi,nlhi->nlh", Q, K.cumsum(1))`` (``causal_linear_attention.py:95``).
    Forward and backward are native streaming kernels (fp32 accumulation, every tensor read
    once); saves only Q and K."""

    @staticmethod
    def forward(ctx, Q, K):
        den = causal_normaliser_raw(Q.data, K.data)
        ctx.save_for_backward(Q, K)
        return den

    @staticmethod
    def backward(ctx, grad_den):
        Q, K = ctx.saved_tensors
        need_q, need_k = ctx.needs_input_grad
        return causal_normaliser_backward_raw(Q.data, K.data, grad_den, need_q, need_k)


causal_normaliser = CausalNormaliser.apply
