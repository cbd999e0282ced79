"""Feature maps phi applied to queries and keys before the causal product.

Mirror of ``fast_transformers/feature_maps``: the ``FeatureMap`` interface and
``elu_feature_map`` (``base.py:19-73``), and the positive orthogonal random features
``Favor`` with its base ``RandomFourierFeatures`` (``fourier_features.py:19-113,165-243``).
An attention layer receives a FACTORY: a callable taking the query dimensionality and
returning the map instance (``base.py:44-54``).
"""
from math import log, sqrt
import warnings

import torch
from torch.nn import Module


class FeatureMap(Module):
    def __init__(self, query_dims):
        super().__init__()
        self.query_dims = query_dims

    def new_feature_map(self, device):
        """Resample the parameters of a random map (no-op for deterministic maps)."""
        raise NotImplementedError()

    def forward_queries(self, x):
        return self(x)

    def forward_keys(self, x):
        return self(x)

    def forward(self, x):
        raise NotImplementedError()

    @classmethod
    def factory(cls, *args, **kwargs):
        def inner(query_dims):
            return cls(query_dims, *args, **kwargs)
        return inner


class ActivationFunctionFeatureMap(FeatureMap):
    """phi(x) = f(x) element-wise."""

    def __init__(self, query_dims, activation_function):
        super().__init__(query_dims)
        self.activation_function = activation_function

    def new_feature_map(self, device):
        return

    def forward(self, x):
        return self.activation_function(x)


def _elu_plus_one(x):
    return torch.nn.functional.elu(x) + 1


elu_feature_map = ActivationFunctionFeatureMap.factory(_elu_plus_one)
# marker the fused layer kernel keys on: this activation can be applied on load
_elu_plus_one.fused_id = "elu+1"


def elu_plus_one_forward_raw(xc, w):
    """``(elu(xc) + 1) * w`` in one native pass, no autograd: ``xc`` contiguous, float32 or
    bfloat16 on CUDA; ``w`` None or a contiguous float32 tensor with one weight per leading row."""
    import ctypes
    from .. import _native
    y = torch.empty_like(xc)
    per = xc.numel() // w.numel() if w is not None and w.numel() else 1
    with torch.cuda.device(xc.device):
        st = _native.lib().ftb_elu_feature_map(
            ctypes.c_void_p(xc.data_ptr()), ctypes.c_void_p(y.data_ptr()),
            ctypes.c_void_p(w.data_ptr()) if w is not None else None, xc.numel(), per,
            0 if xc.dtype == torch.float32 else 1,
            ctypes.c_void_p(torch.cuda.current_stream(xc.device).cuda_stream))
    _native.check(st, "ftb_elu_feature_map")
    return y


def elu_plus_one_backward_raw(xc, g, w):
    """``g * w * (xc > 0 ? 1 : exp(xc))``: the gradient of ``elu_plus_one_forward_raw``."""
    import ctypes
    from .. import _native
    g = g.contiguous()
    gx = torch.empty_like(xc)
    per = xc.numel() // w.numel() if w is not None and w.numel() else 1
    with torch.cuda.device(xc.device):
        st = _native.lib().ftb_elu_feature_map_backward(
            ctypes.c_void_p(xc.data_ptr()), ctypes.c_void_p(g.data_ptr()),
            ctypes.c_void_p(gx.data_ptr()),
            ctypes.c_void_p(w.data_ptr()) if w is not None else None, xc.numel(), per,
            0 if xc.dtype == torch.float32 else 1,
            ctypes.c_void_p(torch.cuda.current_stream(xc.device).cuda_stream))
    _native.check(st, "ftb_elu_feature_map_backward")
    return gx


class _EluPlusOneNative(torch.autograd.Function):
    """``(elu(x) + 1) * w`` with ``w`` one weight per leading-dimension row (or none) in one native
    pass, gradient ``g * w * (x > 0 ? 1 : exp(x))`` in another: the default feature map with the
    layer's key-length mask folded in (``feature_maps/base.py:71-73``,
    ``attention/causal_linear_attention.py:83``)."""

    @staticmethod
    def forward(ctx, x, weights):
        xc = x.contiguous()
        w = None if weights is None else weights.to(torch.float32).contiguous()
        y = elu_plus_one_forward_raw(xc, w)
        ctx.save_for_backward(xc, w)
        return y

    @staticmethod
    def backward(ctx, grad_y):
        xc, w = ctx.saved_tensors
        return elu_plus_one_backward_raw(xc, grad_y, w), None


def elu_plus_one_native(x, row_weights=None):
    """``(elu(x) + 1) * row_weights[..., None, None]`` for a CUDA tensor ``x`` of float32 or
    bfloat16; ``row_weights`` has the shape of ``x``'s leading dimensions (for (N, S, H, E) keys
    the (N, S) key-length mask) or is None."""
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("elu_plus_one_native needs a float32 or bfloat16 CUDA tensor")
    if row_weights is not None and (
            row_weights.dim() > x.dim() or
            tuple(row_weights.shape) != tuple(x.shape[:row_weights.dim()])):
        # the reference's K * float_matrix[:, :, None, None] fails to broadcast in this case
        raise RuntimeError("row_weights of shape %r does not match the leading dimensions of x %r"
                           % (tuple(row_weights.shape), tuple(x.shape)))
    return _EluPlusOneNative.apply(x, row_weights)


def is_default_elu_map(feature_map):
    """True for the default map phi(x) = elu(x) + 1, which the native kernels apply themselves."""
    f = getattr(feature_map, "activation_function", None)
    return getattr(f, "fused_id", None) == "elu+1"


def orthogonal_random_matrix_(w):
    """Fill ``w`` (rows x columns) in place with blocks of ``rows`` orthogonal columns whose
    norms follow the chi distribution with ``rows`` degrees of freedom
    (``fourier_features.py:19-41``): QR of a Gaussian block, columns rescaled by the norms
    of the block's rows."""
    rows, columns = w.shape
    for start in range(0, columns, rows):
        end = min(start + rows, columns)
        block = torch.randn(rows, rows, device=w.device)
        norms = block.pow(2).sum(dim=1).sqrt()
        Q, _ = torch.linalg.qr(block)
        w[:, start:end] = Q[:, :end - start] * norms[None, :end - start]


class RandomFourierFeatures(FeatureMap):
    """[cos(x w), sin(x w)] * sqrt(2 / n_dims) with x scaled by softmax_temp^(1/2)
    (``fourier_features.py:44-113``).  Holds the buffer ``omega`` (query_dims x n_dims/2),
    resampled by ``new_feature_map`` every ``redraw`` calls, never in eval mode when
    ``deterministic_eval``."""

    def __init__(self, query_dimensions, n_dims=None, softmax_temp=None, orthogonal=False,
                 redraw=1, deterministic_eval=False):
        super().__init__(query_dimensions)
        self.n_dims = n_dims or query_dimensions
        self.query_dimensions = query_dimensions
        self.orthogonal = orthogonal
        self.softmax_temp = 1 / sqrt(query_dimensions) if softmax_temp is None else softmax_temp
        self.redraw = redraw
        self.deterministic_eval = deterministic_eval
        self.register_buffer("omega", torch.zeros(self.query_dimensions, self.n_dims // 2))
        self._calls = -1

    def new_feature_map(self, device):
        if self.deterministic_eval and not self.training:
            return
        self._calls += 1
        if (self._calls % self.redraw) != 0:
            return
        omega = torch.zeros(self.query_dimensions, self.n_dims // 2, device=device)
        if self.orthogonal:
            orthogonal_random_matrix_(omega)
        else:
            omega.normal_()
        self.register_buffer("omega", omega)

    def forward(self, x):
        x = x * sqrt(self.softmax_temp)
        u = x.unsqueeze(-2).matmul(self.omega).squeeze(-2)
        phi = torch.cat([torch.cos(u), torch.sin(u)], dim=-1)
        return phi * sqrt(2 / self.n_dims)


class Favor(RandomFourierFeatures):
    """Positive random features approximating the softmax kernel
    (``fourier_features.py:165-243``): with x <- x * softmax_temp^(1/2), u = x omega and
    offset = |x|^2 / 2 + log(n_dims) / 2 (plus, when ``stabilize``, the maximum of |x|^2 over
    the sequence axis), phi(x) = [exp(u - offset), exp(-u - offset)]."""

    def __init__(self, query_dimensions, n_dims=None, softmax_temp=None, orthogonal=True,
                 stabilize=False, redraw=1, deterministic_eval=False):
        super().__init__(query_dimensions, n_dims=n_dims, softmax_temp=softmax_temp,
                         orthogonal=orthogonal, redraw=redraw,
                         deterministic_eval=deterministic_eval)
        self.stabilize = stabilize

    def _check_sequence_length(self, x):
        if len(x.shape) != 4:
            warnings.warn("Favor.stabilize is set to True but the input feature does not have "
                          "the shape (N, L, H, D) which may result in unexpected behaviour")
        if x.shape[1] < x.shape[2]:
            warnings.warn("Favor.stabilize is set to True but the 2nd dimension of the input is "
                          "smaller than the 3rd which could indicate that the sequence length "
                          "and the heads are flipped. The shape of the input is "
                          "{!r}.".format(x.shape))

    def _omega_transposed(self):
        """omega^T as the native forward reads it, made once per draw of omega (the buffer is
        redrawn in place, which bumps its version counter)."""
        key = (self.omega.data_ptr(), self.omega._version)
        if getattr(self, "_omega_t_key", None) != key:
            self._omega_t = self.omega.detach().t().contiguous()
            self._omega_t_key = key
        return self._omega_t

    def forward(self, x):
        from ..settings import get_mode
        if (not self.stabilize and x.is_cuda and x.dtype == torch.float32 and get_mode() == "mma"
                and x.shape[-1] == 64 and self.n_dims in (128, 256) and x.numel() > 0
                and self.omega.device == x.device and self.omega.dtype == torch.float32):
            # tensor-core mode: the whole map as one native pass (TF32 product, like that mode's
            # attention kernels); the reference's formulation below stays the fp32-mode path
            return _FavorNative.apply(x, self.omega, float(self.softmax_temp), self._omega_transposed())
        x = x * sqrt(self.softmax_temp)
        norm_x_squared = torch.einsum("...d,...d->...", x, x).unsqueeze(-1)
        u = x.unsqueeze(-2).matmul(self.omega).squeeze(-2)
        offset = norm_x_squared * 0.5 + 0.5 * log(self.n_dims)
        if self.stabilize:
            self._check_sequence_length(norm_x_squared)
            offset = offset + norm_x_squared.max(1, keepdim=True)[0]
        return torch.cat([torch.exp(u - offset), torch.exp(-u - offset)], dim=-1)


def favor_features_raw(x, omega, softmax_temp, omega_t=None):
    """``[exp(u - off), exp(-u - off)]`` with ``u = x temp^(1/2) omega``, ``off = |x|^2 temp / 2 +
    log(n) / 2`` (``fourier_features.py:218-243``) in one native pass: ``x`` (..., 64) float32 on
    CUDA, ``omega`` (64, n/2) with n/2 = 64 or 128.  No autograd."""
    import ctypes
    from .. import _native
    xc = x.contiguous()
    half = omega.shape[1]
    rows = xc.numel() // xc.shape[-1]
    if omega_t is None:
        omega_t = omega.t().contiguous()
    out = torch.empty(xc.shape[:-1] + (2 * half,), device=xc.device, dtype=torch.float32)
    with torch.cuda.device(xc.device):
        st = _native.lib().ftb_favor_feature_map(
            ctypes.c_void_p(xc.data_ptr()), ctypes.c_void_p(omega_t.data_ptr()),
            ctypes.c_void_p(out.data_ptr()), rows, xc.shape[-1], half, xc.shape[-1], 2 * half,
            float(softmax_temp), ctypes.c_void_p(torch.cuda.current_stream(xc.device).cuda_stream))
    _native.check(st, "ftb_favor_feature_map")
    return out


def favor_features_backward_raw(grad_phi, phi, x, omega, softmax_temp):
    """The input gradient of ``favor_features_raw`` in one native pass
    (``ftb_favor_feature_map_backward``).  No autograd."""
    import ctypes
    from .. import _native
    g, xc = grad_phi.contiguous(), x.contiguous()
    half = omega.shape[1]
    rows = xc.numel() // xc.shape[-1]
    om = omega.contiguous()
    grad_x = torch.empty_like(xc)
    vp = ctypes.c_void_p
    with torch.cuda.device(xc.device):
        st = _native.lib().ftb_favor_feature_map_backward(
            vp(g.data_ptr()), vp(phi.data_ptr()), vp(xc.data_ptr()), vp(om.data_ptr()), vp(grad_x.data_ptr()),
            rows, xc.shape[-1], half, 2 * half, 2 * half, xc.shape[-1], xc.shape[-1], float(softmax_temp),
            vp(torch.cuda.current_stream(xc.device).cuda_stream))
    _native.check(st, "ftb_favor_feature_map_backward")
    return grad_x


class _FavorNative(torch.autograd.Function):
    """Favor's feature map, forward and backward one native pass each on the tensor cores.  The
    backward is the chain rule on the saved input and OUTPUT -- with phi = [p, m]:
    ``grad_u = g_p * p - g_m * m``, ``grad_off = -sum(g * phi)``,
    ``grad_x = temp^(1/2) * (grad_u omega^T) + temp * grad_off * x``."""

    @staticmethod
    def forward(ctx, x, omega, softmax_temp, omega_t=None):
        phi = favor_features_raw(x, omega, softmax_temp, omega_t)
        ctx.save_for_backward(x, omega, phi)
        ctx.softmax_temp = softmax_temp
        return phi

    @staticmethod
    def backward(ctx, grad_phi):
        x, omega, phi = ctx.saved_tensors
        half = omega.shape[1]
        if grad_phi.dtype == torch.float32 and grad_phi.is_cuda:
            return favor_features_backward_raw(grad_phi, phi, x, omega, ctx.softmax_temp), None, None, None
        gp = grad_phi * phi
        grad_u = gp[..., :half] - gp[..., half:]
        grad_off = -gp.sum(dim=-1, keepdim=True)
        grad_x = sqrt(ctx.softmax_temp) * grad_u.matmul(omega.t()) + ctx.softmax_temp * grad_off * x
        return grad_x, None, None, None
