"""CPU oracle for the causal linear-attention hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module: it is the checker used by ``tests/``,
by ``__graft_entry__.smoke()`` and by the CPU-baseline / reference arm of ``bench.py``.

Parity status: PINNED.  The reference ships no stored known-answer vectors for this path
(its tests compare against a dense PyTorch form on fresh random inputs), so the pins are
(1) outputs of the unmodified reference CPU extension, compiled by ``oracle/build_ref.py``
and run on seeded inputs, committed under ``tests/golden/`` together with the generating
script, and (2) the reference tests' own dense restatement
(``tests/causal_product/test_causal_product_cpu.py:32-74``), reproduced here in fp64.

Functions (each cites the reference lines it restates):

* ``dense_forward`` / ``dense_backward``      -- masked ``tril(Q K^T) V`` and its autograd,
  the form the reference tests use as ground truth.
* ``chunked_forward`` / ``chunked_backward``  -- the same maths as an fp64 blocked
  recurrence, for sequence lengths where an L x L matrix is too large.
* ``c_forward`` / ``c_backward``              -- ``oracle/causal_oracle.c`` via ctypes: the
  sequential recurrence of ``causal_product_cpu.cpp:82-209`` in fp32 or fp64 accumulation.
* ``reference_ext``                           -- the compiled reference extension itself.
* ``layer_forward``                           -- ``CausalLinearAttention.forward``
  (``fast_transformers/attention/causal_linear_attention.py:71-104``) restated densely.
* ``linear_layer_forward`` / ``linear_product`` -- the unmasked ``LinearAttention.forward``
  (``fast_transformers/attention/linear_attention.py:55-80``) and its numerator.
* ``favor_features`` / ``elu_features``       -- the two feature maps on the path
  (``feature_maps/base.py:71-73``, ``feature_maps/fourier_features.py:218-243``).
"""
import ctypes
import importlib.machinery
import importlib.util
import math
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


# ----------------------------------------------------------------------------------------
# error metric
# ----------------------------------------------------------------------------------------
def rel_err(x, ref):
    """max|x - ref| / max|ref| -- the metric the stated tolerances (1e-5 / 2e-2) refer to."""
    x = torch.as_tensor(x).double().cpu()
    ref = torch.as_tensor(ref).double().cpu()
    denom = ref.abs().max().item()
    return (x - ref).abs().max().item() / (denom if denom > 0 else 1.0)


def max_relative_error(a, b, eps=1e-6):
    """Element-wise relative error of the reference's own tests
    (``tests/causal_product/test_causal_product_cpu.py:19-20``)."""
    a = torch.as_tensor(a).double().cpu()
    b = torch.as_tensor(b).double().cpu()
    return torch.abs((a - b) / (torch.abs(a) + eps)).max().item()


# ----------------------------------------------------------------------------------------
# dense form (reference tests' ground truth), fp64
# ----------------------------------------------------------------------------------------
def dense_forward(Q, K, V, dtype=torch.float64):
    """``einsum("nhls,nhsm,ls->nhlm", Q K^T, V, tril)`` -- test_causal_product_cpu.py:45-47."""
    Q, K, V = (t.detach().to("cpu", dtype) for t in (Q, K, V))
    L = Q.shape[2]
    A = torch.einsum("nhle,nhse->nhls", Q, K)
    A = A * torch.tril(torch.ones(L, L, dtype=dtype))
    return torch.einsum("nhls,nhsm->nhlm", A, V)


def dense_backward(Q, K, V, G, dtype=torch.float64):
    """Gradients of ``sum(out * G)`` by autograd through the dense form --
    test_causal_product_cpu.py:63-70."""
    Q, K, V, G = (t.detach().to("cpu", dtype) for t in (Q, K, V, G))
    Q.requires_grad_(True), K.requires_grad_(True), V.requires_grad_(True)
    L = Q.shape[2]
    A = torch.einsum("nhle,nhse->nhls", Q, K) * torch.tril(torch.ones(L, L, dtype=dtype))
    out = torch.einsum("nhls,nhsm->nhlm", A, V)
    (out * G).sum().backward()
    return Q.grad, K.grad, V.grad


# ----------------------------------------------------------------------------------------
# blocked recurrence, fp64, for long sequences
# ----------------------------------------------------------------------------------------
def chunked_forward(Q, K, V, chunk=256, dtype=torch.float64, initial_state=None,
                    return_state=False):
    """out_i = q_i . S_i with S_i = S_init + sum_{j<=i} k_j v_j^T, evaluated block by block
    (causal_product_cpu.cpp:106-121 regrouped; algebraically identical)."""
    Q, K, V = (t.detach().to("cpu", dtype) for t in (Q, K, V))
    N, H, L, D = Q.shape
    M = V.shape[3]
    S = torch.zeros(N, H, D, M, dtype=dtype) if initial_state is None \
        else initial_state.detach().to("cpu", dtype).clone()
    out = torch.empty(N, H, L, M, dtype=dtype)
    for s in range(0, L, chunk):
        e = min(L, s + chunk)
        q, k, v = Q[:, :, s:e], K[:, :, s:e], V[:, :, s:e]
        P = torch.tril(q @ k.transpose(-1, -2))
        out[:, :, s:e] = q @ S + P @ v
        S = S + k.transpose(-1, -2) @ v
    return (out, S) if return_state else out


def chunked_backward(Q, K, V, G, chunk=256, dtype=torch.float64, initial_state=None,
                     final_grad_state=None):
    """gq_i = S_i g_i (l ascending), gk_i = R_i v_i and gv_i = R_i^T k_i with
    R_i = R_final + sum_{j>=i} q_j g_j^T (l descending) -- causal_product_cpu.cpp:165-206."""
    Q, K, V, G = (t.detach().to("cpu", dtype) for t in (Q, K, V, G))
    N, H, L, D = Q.shape
    M = V.shape[3]
    gQ, gK, gV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
    S = torch.zeros(N, H, D, M, dtype=dtype) if initial_state is None \
        else initial_state.detach().to("cpu", dtype).clone()
    for s in range(0, L, chunk):
        e = min(L, s + chunk)
        k, v, g = K[:, :, s:e], V[:, :, s:e], G[:, :, s:e]
        W = torch.tril(g @ v.transpose(-1, -2))
        gQ[:, :, s:e] = g @ S.transpose(-1, -2) + W @ k
        S = S + k.transpose(-1, -2) @ v
    R = torch.zeros(N, H, D, M, dtype=dtype) if final_grad_state is None \
        else final_grad_state.detach().to("cpu", dtype).clone()
    starts = list(range(0, L, chunk))
    for s in reversed(starts):
        e = min(L, s + chunk)
        q, k, v, g = Q[:, :, s:e], K[:, :, s:e], V[:, :, s:e], G[:, :, s:e]
        W = torch.tril(g @ v.transpose(-1, -2))      # W[i, j] = g_i . v_j, j <= i
        P = torch.tril(q @ k.transpose(-1, -2))      # P[i, j] = q_i . k_j, j <= i
        gK[:, :, s:e] = v @ R.transpose(-1, -2) + W.transpose(-1, -2) @ q
        gV[:, :, s:e] = k @ R + P.transpose(-1, -2) @ g
        R = R + q.transpose(-1, -2) @ g
    return gQ, gK, gV


def local_states(Q, K, V, G=None, dtype=torch.float64):
    """Whole-range sums K^T V (and Q^T G): what one sequence shard contributes to the
    running states of the shards after (before) it."""
    K, V = K.detach().to("cpu", dtype), V.detach().to("cpu", dtype)
    S = K.transpose(-1, -2) @ V
    if G is None:
        return S
    Q, G = Q.detach().to("cpu", dtype), G.detach().to("cpu", dtype)
    return S, Q.transpose(-1, -2) @ G


# ----------------------------------------------------------------------------------------
# the C restatement (sequential recurrence, reference summation order)
# ----------------------------------------------------------------------------------------
_clib = None


def _c():
    global _clib
    if _clib is None:
        path = os.path.join(HERE, "libcausal_oracle_c.so")
        if not os.path.exists(path):
            import sys
            sys.path.insert(0, HERE)
            try:
                import build_ref
            finally:
                sys.path.pop(0)
            build_ref.build_c_oracle()
        _clib = ctypes.CDLL(path)
    return _clib


def _i64(seq):
    return (ctypes.c_int64 * len(seq))(*seq)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _check(t):
    assert t.device.type == "cpu" and t.dim() == 4 and t.stride(3) == 1


def c_forward(Q, K, V, acc="f32"):
    """Run ``causal_oracle_forward_{f32,f64}``; fp32 inputs, any batch/head/row strides."""
    Q, K, V = (t.detach().float() for t in (Q, K, V))
    for t in (Q, K, V):
        _check(t)
    N, H, L, D = Q.shape
    M = V.shape[3]
    out = torch.zeros(N, H, L, M, dtype=torch.float32 if acc == "f32" else torch.float64)
    fn = getattr(_c(), "causal_oracle_forward_" + acc)
    fn(_p(Q), _p(K), _p(V), _p(out), *(ctypes.c_int64(x) for x in (N, H, L, D, M)),
       _i64(Q.stride()[:3]), _i64(K.stride()[:3]), _i64(V.stride()[:3]),
       _i64(out.stride()[:3]))
    return out


def c_backward(Q, K, V, G, acc="f32"):
    Q, K, V, G = (t.detach().float() for t in (Q, K, V, G))
    G = G.contiguous()
    for t in (Q, K, V, G):
        _check(t)
    N, H, L, D = Q.shape
    M = V.shape[3]
    dt = torch.float32 if acc == "f32" else torch.float64
    gQ = torch.zeros(N, H, L, D, dtype=dt)
    gK = torch.zeros(N, H, L, D, dtype=dt)
    gV = torch.zeros(N, H, L, M, dtype=dt)
    fn = getattr(_c(), "causal_oracle_backward_" + acc)
    fn(_p(Q), _p(K), _p(V), _p(G), _p(gQ), _p(gK), _p(gV),
       *(ctypes.c_int64(x) for x in (N, H, L, D, M)),
       _i64(Q.stride()[:3]), _i64(K.stride()[:3]), _i64(V.stride()[:3]),
       _i64(G.stride()[:3]), _i64(gQ.stride()[:3]), _i64(gK.stride()[:3]),
       _i64(gV.stride()[:3]))
    return gQ, gK, gV


# ----------------------------------------------------------------------------------------
# the compiled reference extension (oracle/_ref)
# ----------------------------------------------------------------------------------------
_ref_mod = None


def reference_ext():
    """The reference's own ``causal_product_cpu`` module (functions ``causal_dot_product``
    and ``causal_dot_backward``, in-place outputs -- causal_product_cpu.cpp:212-225), or
    None if it has not been built."""
    global _ref_mod
    if _ref_mod is None:
        path = os.path.join(HERE, "_ref", "causal_product_cpu.so")
        if not os.path.exists(path):
            return None
        loader = importlib.machinery.ExtensionFileLoader("causal_product_cpu", path)
        spec = importlib.util.spec_from_loader("causal_product_cpu", loader)
        mod = importlib.util.module_from_spec(spec)
        loader.exec_module(mod)
        _ref_mod = mod
    return _ref_mod


def reference_forward(Q, K, V):
    ext = reference_ext()
    out = torch.zeros(Q.shape[0], Q.shape[1], Q.shape[2], V.shape[3])
    ext.causal_dot_product(Q, K, V, out)
    return out


def reference_backward(Q, K, V, G):
    ext = reference_ext()
    gQ, gK, gV = torch.zeros_like(Q), torch.zeros_like(K), torch.zeros_like(V)
    ext.causal_dot_backward(Q, K, V, G, gQ, gK, gV)
    return gQ, gK, gV


# ----------------------------------------------------------------------------------------
# feature maps and the layer, restated densely
# ----------------------------------------------------------------------------------------
def elu_features(x):
    """phi(x) = elu(x) + 1 -- feature_maps/base.py:71-73."""
    return torch.nn.functional.elu(x) + 1


def favor_features(x, omega, softmax_temp=None, stabilize=False):
    """Positive random features of Favor.forward (fourier_features.py:218-243):
    x <- x * temp^(1/2); u = x omega; offset = |x|^2/2 + log(n_dims)/2
    (+ max over the sequence axis of |x|^2 when ``stabilize``); phi = [e^(u-off), e^(-u-off)]."""
    E = x.shape[-1]
    n_dims = 2 * omega.shape[1]
    temp = 1.0 / math.sqrt(E) if softmax_temp is None else softmax_temp
    x = x * math.sqrt(temp)
    nx2 = (x * x).sum(-1, keepdim=True)
    u = x @ omega.to(x.dtype)
    off = 0.5 * nx2 + 0.5 * math.log(n_dims)
    if stabilize:
        off = off + nx2.max(1, keepdim=True)[0]
    return torch.cat([torch.exp(u - off), torch.exp(-u - off)], dim=-1)


def layer_forward(queries, keys, values, key_lengths=None, feature=elu_features, eps=1e-6,
                  dtype=torch.float64):
    """``CausalLinearAttention.forward`` for a lower-triangular mask
    (causal_linear_attention.py:71-104): inputs (N, L, H, E), (N, S, H, E), (N, S, H, M);
    K is multiplied by the key-length mask (:83), sliced or zero-padded to L (:57-69);
    Z = 1 / (Q . cumsum(K) + eps) (:95); result (N, L, H, M)."""
    q = feature(queries.detach().to("cpu", dtype))
    k = feature(keys.detach().to("cpu", dtype))
    v = values.detach().to("cpu", dtype)
    N, L, H, _ = q.shape
    S = k.shape[1]
    if key_lengths is not None:
        mask = (torch.arange(S)[None, :] < key_lengths.cpu()[:, None]).to(dtype)
        k = k * mask[:, :, None, None]
    if L < S:
        k, v = k[:, :L], v[:, :L]
    elif L > S:
        k = torch.cat([k, k.new_zeros(N, L - S, H, k.shape[3])], dim=1)
        v = torch.cat([v, v.new_zeros(N, L - S, H, v.shape[3])], dim=1)
    Z = 1.0 / (torch.einsum("nlhi,nlhi->nlh", q, k.cumsum(1)) + eps)
    A = torch.einsum("nlhe,nshe->nhls", q, k) * torch.tril(torch.ones(L, L, dtype=dtype))
    out = torch.einsum("nhls,nshm->nlhm", A, v)
    return out * Z[:, :, :, None]


def linear_layer_forward(queries, keys, values, key_lengths=None, feature=elu_features, eps=1e-6,
                         dtype=torch.float64):
    """``LinearAttention.forward`` (fast_transformers/attention/linear_attention.py:55-80), the
    unmasked form: inputs (N, L, H, E), (N, S, H, E), (N, S, H, M); K is multiplied by the
    key-length mask (:68); KV = sum_s K_s (x) v_s (:73); Z = 1 / (Q . sum_s K_s + eps) (:76);
    result (N, L, H, M) = (Q . KV) Z (:79)."""
    q = feature(queries.detach().to("cpu", dtype))
    k = feature(keys.detach().to("cpu", dtype))
    v = values.detach().to("cpu", dtype)
    S = k.shape[1]
    if key_lengths is not None:
        mask = (torch.arange(S)[None, :] < key_lengths.cpu()[:, None]).to(dtype)
        k = k * mask[:, :, None, None]
    KV = torch.einsum("nshd,nshm->nhdm", k, v)
    Z = 1.0 / (torch.einsum("nlhd,nhd->nlh", q, k.sum(dim=1)) + eps)
    return torch.einsum("nlhd,nhdm,nlh->nlhm", q, KV, Z)


def linear_product(Q, K, V, G=None, dtype=torch.float64):
    """The unmasked product out = Q (K^T V) for (N, H, L, D), (N, H, S, D), (N, H, S, M) tensors
    (the two einsums of linear_attention.py:73,79 without the normaliser) and, with ``G``, its
    gradients by autograd.  Returns out or (out, gQ, gK, gV)."""
    Q, K, V = (t.detach().to("cpu", dtype) for t in (Q, K, V))
    if G is None:
        return Q @ (K.transpose(-1, -2) @ V)
    Q.requires_grad_(True), K.requires_grad_(True), V.requires_grad_(True)
    out = Q @ (K.transpose(-1, -2) @ V)
    (out * G.detach().to("cpu", dtype)).sum().backward()
    return out.detach(), Q.grad, K.grad, V.grad


def normaliser(Q, K, dtype=torch.float64):
    """``den[n,h,l] = Q[n,h,l] . sum_{j<=l} K[n,h,j]`` for (N, H, L, D) tensors -- the argument of
    the reciprocal in causal_linear_attention.py:95 (there in (N, L, H, D) layout)."""
    q = Q.detach().to("cpu", dtype)
    k = K.detach().to("cpu", dtype)
    return torch.einsum("nhld,nhld->nhl", q, k.cumsum(2))


def recurrent_step(query, key, value, state=None, feature=elu_features, eps=1e-6,
                   dtype=torch.float64):
    """One step of ``RecurrentLinearAttention.forward``
    (recurrent/attention/self_attention/linear_attention.py:55-90): inputs (N, H, E),
    (N, H, E), (N, H, M) and the state ``[S (N,H,E,M), z (N,H,E)]`` or None (zeros, :64-67);
    ``z += K; S += K (x) v`` (:78-83), ``Z = 1 / (Q . z + eps)``, ``y = (Q . S) Z`` (:86-87).
    Returns ``(y, [S, z])`` in ``dtype``; the inputs are not modified."""
    Q = feature(query.detach().to("cpu", dtype))
    K = feature(key.detach().to("cpu", dtype))
    v = value.detach().to("cpu", dtype)
    N, H, E = Q.shape
    if state is None:
        S = Q.new_zeros(N, H, E, v.shape[2])
        z = Q.new_zeros(N, H, E)
    else:
        S, z = (t.detach().to("cpu", dtype).clone() for t in state)
    z = z + K
    S = S + torch.einsum("nhd,nhm->nhdm", K, v)
    Z = 1.0 / (torch.einsum("nhd,nhd->nh", Q, z) + eps)
    return torch.einsum("nhd,nhdm,nh->nhm", Q, S, Z), [S, z]


def to_numpy(*ts):
    return [np.asarray(t.detach().cpu()) for t in ts]
