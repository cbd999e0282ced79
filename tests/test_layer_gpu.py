"""CausalLinearAttention, AttentionLayer and the encoder on the GPU against the
reference's outputs (golden fixtures) and the dense fp64 oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import causal_oracle as orc  # noqa: E402
from fast_transformers_b200.attention import CausalLinearAttention  # noqa: E402
from fast_transformers_b200.builders import TransformerEncoderBuilder  # noqa: E402
from fast_transformers_b200.feature_maps import Favor  # noqa: E402
from fast_transformers_b200.masking import LengthMask, TriangularCausalMask  # noqa: E402


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available()
    return native_lib


def T(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("case", ["eq", "lt", "gt"])
def test_layer_matches_reference(golden, case):
    g = golden("layer")
    q, k, v, w = (T(g[case + "_" + n]).cuda() for n in "qkvw")
    klen = T(g[case + "_klen"]).cuda()
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    N, L = q.shape[:2]
    S = k.shape[1]
    att = CausalLinearAttention(q.shape[3])
    y = att(q, k, v, TriangularCausalMask(L, device="cuda"),
            LengthMask(torch.full((N,), L, device="cuda")), LengthMask(klen, max_len=S))
    assert y.is_contiguous() and y.shape == (N, L, q.shape[2], v.shape[3])
    # the reference's own bound for the normalised product (test_causal_product.py:54-62)
    assert (y.cpu() - T(g[case + "_y"])).abs().max() < 5e-4
    assert orc.rel_err(y, orc.layer_forward(q, k, v, key_lengths=klen)) < 1e-5
    (y * w).sum().backward()
    if case != "gt":
        for n, t in (("gq", q), ("gk", k), ("gv", v)):
            assert (t.grad.cpu() - T(g[case + "_" + n])).abs().max() < 5e-4, n
    else:
        assert v.grad.shape == v.shape and torch.isfinite(v.grad).all()


def test_layer_with_favor_map():
    torch.manual_seed(3)
    N, L, H, E, M = 2, 50, 3, 16, 8
    q, k, v = (torch.randn(N, L, H, d, device="cuda") * 0.5 for d in (E, E, M))
    att = CausalLinearAttention(E, feature_map=Favor.factory(n_dims=64, redraw=10 ** 9)).cuda()
    lm = LengthMask(torch.full((N,), L, device="cuda"))
    y = att(q, k, v, TriangularCausalMask(L, device="cuda"), lm, lm)
    omega = att.feature_map.omega.double().cpu()
    want = orc.layer_forward(q, k, v, feature=lambda x: orc.favor_features(x, omega))
    assert orc.rel_err(y, want) < 1e-5


def test_encoder_matches_reference(golden):
    g = golden("encoder")
    model = TransformerEncoderBuilder.from_kwargs(
        n_layers=2, n_heads=4, query_dimensions=8, value_dimensions=8,
        feed_forward_dimensions=64, attention_type="causal-linear", dropout=0.0).get()
    model.load_state_dict({k[4:]: T(g[k]) for k in g.files if k.startswith("sd__")})
    model = model.cuda()
    x = T(g["x"]).cuda().requires_grad_(True)
    with pytest.raises(RuntimeError):
        model(x)  # the default full mask is rejected, as in the reference
    y = model(x, attn_mask=TriangularCausalMask(40, device="cuda"))
    assert (y.cpu() - T(g["y"])).abs().max() < 1e-4
    (y * T(g["w"]).cuda()).sum().backward()
    assert orc.rel_err(x.grad, T(g["gx"])) < 1e-3
    for name, p in model.named_parameters():
        ref = T(g["gp__" + name])
        assert (p.grad.cpu() - ref).abs().max() <= 1e-3 * max(1.0, ref.abs().max().item()), name


def test_encoder_tensor_core_mode_close_to_reference():
    """The same encoder in the tensor-core mode (TF32 attention products): within the 2e-2 tier of
    the reference's fp32 output."""
    import fast_transformers_b200 as ftb
    model = TransformerEncoderBuilder.from_kwargs(
        n_layers=2, n_heads=4, query_dimensions=64, value_dimensions=64,
        feed_forward_dimensions=64, attention_type="causal-linear", dropout=0.0).get().cuda()
    torch.manual_seed(0)
    x = torch.rand(2, 300, 256, device="cuda", requires_grad=True)
    mask = TriangularCausalMask(300, device="cuda")
    # the encoder ends in a LayerNorm, so sum(y) and sum(y^2) are constants: weight the output
    w = torch.randn(2, 300, 256, device="cuda")
    with ftb.mode("fp32"):
        y32 = model(x, attn_mask=mask)
        (g32,) = torch.autograd.grad((y32 * w).sum(), x)
    with ftb.mode("mma"):
        ym = model(x, attn_mask=mask)
        (gm,) = torch.autograd.grad((ym * w).sum(), x)
    assert orc.rel_err(ym, y32) < 2e-2
    # The 2e-2 tier is stated for the product.  Through the layer the gradient of num/Z is a
    # difference of two nearly equal terms (the normalised output is a weighted mean of the
    # values), one rounded to TF32 and one not, and two layers compound it: measured 3.3e-2.
    assert orc.rel_err(gm, g32) < 1e-1
    assert not torch.equal(ym, y32)   # the two modes really are different code paths


@pytest.mark.parametrize("shape", [(2, 3, 333, 64), (1, 2, 5000, 16), (3, 1, 31, 100), (1, 1, 1, 1),
                                   (2, 2, 700, 256), (1, 2, 1000, 128), (2, 1, 257, 32),
                                   (16, 8, 2048, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_native_normaliser_against_fp64(shape, dtype):
    """den = Q . cumsum(K) and its gradients (causal_linear_attention.py:95 and its autograd) from
    the streaming kernels, on (N, L, H, E) storage viewed as (N, H, L, E), one and several
    segments per sequence."""
    from fast_transformers_b200.causal_product import causal_normaliser
    N, H, L, E = shape
    g = torch.Generator().manual_seed(L)
    qs = torch.rand(N, L, H, E, generator=g).to(dtype)
    ks = torch.rand(N, L, H, E, generator=g).to(dtype)
    w = torch.randn(N, H, L, generator=g).to(dtype)
    q = qs.cuda().permute(0, 2, 1, 3).requires_grad_(True)
    k = ks.cuda().permute(0, 2, 1, 3).requires_grad_(True)
    den = causal_normaliser(q, k)
    assert den.shape == (N, H, L) and den.dtype == dtype
    den.backward(w.cuda())
    qd = qs.double().permute(0, 2, 1, 3).requires_grad_(True)
    kd = ks.double().permute(0, 2, 1, 3).requires_grad_(True)
    want = torch.einsum("nhld,nhld->nhl", qd, kd.cumsum(2))
    want.backward(w.double())
    assert orc.rel_err(orc.normaliser(qs.permute(0, 2, 1, 3), ks.permute(0, 2, 1, 3)), want) < 1e-12
    tol = 1e-5 if dtype == torch.float32 else 1e-2     # bf16: rounding of the stored results
    assert orc.rel_err(den, want) < tol
    assert orc.rel_err(q.grad, qd.grad) < tol and orc.rel_err(k.grad, kd.grad) < tol


def test_native_normaliser_partial_gradients_and_limits():
    from fast_transformers_b200 import _native
    from fast_transformers_b200.causal_product import causal_normaliser
    q = torch.rand(1, 2, 300, 32, device="cuda", requires_grad=True)
    k = torch.rand(1, 2, 300, 32, device="cuda")            # no gradient asked for K
    causal_normaliser(q, k).sum().backward()
    want = k.double().cumsum(2)
    assert orc.rel_err(q.grad, want) < 1e-5
    wide = torch.rand(1, 1, 8, 300, device="cuda")
    with pytest.raises(_native.NativeError) as e:
        causal_normaliser(wide, wide)
    assert e.value.status == _native.ERR_UNSUPPORTED
    assert causal_normaliser(torch.rand(0, 2, 5, 4, device="cuda"), torch.rand(0, 2, 5, 4, device="cuda")).shape == (0, 2, 5)


@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.float32, 16), (torch.bfloat16, 128)])
def test_normaliser_gradients_through_the_feature_map_in_place(dtype, D):
    """``ftb_causal_normaliser_backward_elu``: (grad + n) * w * phi'(x) in place equals the
    accumulating normaliser backward followed by the feature map's backward pass."""
    from fast_transformers_b200.causal_product import (causal_normaliser_backward_elu_raw,
                                                       causal_normaliser_backward_raw)
    from fast_transformers_b200.feature_maps import elu_plus_one_backward_raw, elu_plus_one_forward_raw
    g = torch.Generator().manual_seed(D)
    N, L, H = 2, 700, 3
    xq, xk = (torch.randn(N, L, H, D, generator=g).to(dtype).cuda() for _ in range(2))
    w = (torch.arange(L)[None, :] < torch.tensor([L, 400])[:, None]).float().cuda()
    Q, K = elu_plus_one_forward_raw(xq, None), elu_plus_one_forward_raw(xk, w)
    gden = torch.randn(N, L, H, generator=g).cuda().permute(0, 2, 1)
    base = [torch.randn(N, L, H, D, generator=g).to(dtype).cuda() for _ in range(2)]
    P = lambda t: t.permute(0, 2, 1, 3)     # noqa: E731
    want = [b.clone() for b in base]
    causal_normaliser_backward_raw(P(Q), P(K), gden, add_to=(P(want[0]), P(want[1])))
    want = [elu_plus_one_backward_raw(xq, want[0], None), elu_plus_one_backward_raw(xk, want[1], w)]
    got = [b.clone() for b in base]
    assert causal_normaliser_backward_elu_raw(P(Q), P(K), gden, P(got[0]), P(got[1]), P(xq), P(xk), w)
    tol = 1e-6 if dtype == torch.float32 else 2e-2
    for a, b in zip(got, want):
        assert orc.rel_err(a, b.double()) < tol
    # a width the streaming kernels do not take: refused, nothing changed
    odd = [torch.randn(1, 5, 2, 24, device="cuda") for _ in range(6)]
    keep = odd[2].clone()
    assert not causal_normaliser_backward_elu_raw(P(odd[0]), P(odd[1]), torch.randn(1, 2, 5, device="cuda"),
                                                  P(odd[2]), P(odd[3]), P(odd[4]), P(odd[5]))
    assert torch.equal(odd[2], keep)


@pytest.mark.parametrize("M", [16, 64, 128, 24])
def test_division_backward_in_one_pass(M):
    """``grad_out = grad_y Z`` and ``grad_den = -Z sum(grad_y y)`` for ``Z = 1 / (den + eps)`` from one
    native pass (``ftb_normalised_output_grads``; M = 24 takes the torch formulation)."""
    from fast_transformers_b200 import _native
    from fast_transformers_b200.attention.causal_linear_attention import _division_backward
    g = torch.Generator().manual_seed(M)
    N, L, H, eps = 2, 333, 3, 1e-6
    gy, y = (torch.randn(N, L, H, M, generator=g).cuda() for _ in range(2))
    den = (torch.rand(N, L, H, generator=g) * 20 + 0.1).cuda().permute(0, 2, 1)      # (N, H, L) view
    n0 = _native.lib().ftb_launch_count()
    grad_out, grad_den = _division_backward(gy, y, den, eps)
    assert _native.lib().ftb_launch_count() - n0 == (1 if M != 24 else 0)
    Z = 1 / (den.permute(0, 2, 1).double() + eps)
    assert orc.rel_err(grad_out, gy.double() * Z[..., None]) < 1e-6
    assert orc.rel_err(grad_den, -(Z * (gy.double() * y.double()).sum(-1))) < 1e-6


@pytest.mark.parametrize("D,L", [(64, 3000), (128, 700), (40, 333)])
def test_native_normaliser_gradients_added_in_place(D, L):
    """``add_to``: the denominator's gradients are added to tensors that hold other gradients already
    (``ftb_causal_normaliser_backward_add``; the streaming kernels for D = 64 and 128, the tile kernel
    for D = 40), in (N, L, H, D) storage; one of the two may be skipped."""
    from fast_transformers_b200.causal_product import causal_normaliser_backward_raw
    g = torch.Generator().manual_seed(D)
    N, H = 2, 3
    Q, K = (torch.rand(N, L, H, D, generator=g).cuda().permute(0, 2, 1, 3) for _ in range(2))
    gden = torch.randn(N, L, H, generator=g).cuda().permute(0, 2, 1)
    base_q, base_k = (torch.randn(N, L, H, D, generator=g).cuda().permute(0, 2, 1, 3) for _ in range(2))
    nq, nk = causal_normaliser_backward_raw(Q, K, gden)
    aq, ak = base_q.clone(memory_format=torch.preserve_format), base_k.clone(memory_format=torch.preserve_format)
    causal_normaliser_backward_raw(Q, K, gden, add_to=(aq, ak))
    assert torch.equal(aq, base_q + nq) and torch.equal(ak, base_k + nk)
    only_k = base_k.clone(memory_format=torch.preserve_format)
    causal_normaliser_backward_raw(Q, K, gden, add_to=(None, only_k))
    assert torch.equal(only_k, ak)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_native_elu_feature_map_with_key_length_mask(dtype):
    """(elu(x) + 1) * mask and its gradient in one pass each, against torch in fp64
    (feature_maps/base.py:71-73, causal_linear_attention.py:83); odd sizes so that groups of four
    elements straddle mask entries."""
    from fast_transformers_b200.feature_maps import elu_plus_one_native
    g = torch.Generator().manual_seed(31)
    for shape in ((3, 50, 2, 7), (2, 33, 4, 64), (1, 1, 1, 1)):
        x = (torch.randn(shape, generator=g) * 2).to(dtype)
        lengths = torch.randint(1, shape[1] + 1, (shape[0],), generator=g)
        mask = (torch.arange(shape[1])[None, :] < lengths[:, None]).float()
        w = torch.randn(shape, generator=g).to(dtype)
        for m in (None, mask):
            xd = x.cuda().requires_grad_(True)
            y = elu_plus_one_native(xd, None if m is None else m.cuda())
            y.backward(w.cuda())
            x64 = x.double().requires_grad_(True)
            want = torch.nn.functional.elu(x64) + 1
            if m is not None:
                want = want * m.double()[:, :, None, None]
            want.backward(w.double())
            tol = 1e-6 if dtype == torch.float32 else 1e-2
            assert orc.rel_err(y, want) < tol and orc.rel_err(xd.grad, x64.grad) < tol


@pytest.mark.parametrize("mode,dtype", [("fp32", torch.float32), ("mma", torch.float32), ("mma", torch.bfloat16)])
def test_one_node_layer_equals_the_chain_of_nodes(mode, dtype):
    """The layer body as one autograd node (raw inputs kept, feature tensors recomputed in the
    backward) against the chain of separate nodes: same kernels, so the same output bit for bit
    and gradients that differ only by the order of two additions; and against the fp64 oracle."""
    import fast_transformers_b200 as ftb
    from fast_transformers_b200.attention import causal_linear_attention as cla
    g = torch.Generator().manual_seed(33)
    N, L, H, E = 2, 700, 3, 64 if dtype == torch.float32 else 128
    q, k, v, w = (torch.randn(N, L, H, E, generator=g).to(dtype) for _ in range(4))
    klen = torch.tensor([700, 411])
    masks = (TriangularCausalMask(L, device="cuda"), LengthMask(torch.full((N,), L, device="cuda")),
             LengthMask(klen.cuda(), max_len=L))
    att = CausalLinearAttention(E)
    results = []
    for fused in (True, False):
        cla.fused_node_enabled = fused
        try:
            qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
            with ftb.mode(mode):
                y = att(qd, kd, vd, *masks)
                (y * w.cuda()).sum().backward()
            results.append((y.detach(), qd.grad, kd.grad, vd.grad))
        finally:
            cla.fused_node_enabled = True
    tol = 1e-5 if (mode == "fp32" and dtype == torch.float32) else 2e-2
    assert torch.equal(results[0][0], results[1][0])
    for a, b in zip(results[0][1:], results[1][1:]):
        # (bf16: the two forms round their intermediate gradients to bf16 at different points)
        assert orc.rel_err(a, b) < (1e-6 if dtype == torch.float32 else 5e-2)
    want = orc.layer_forward(q.float(), k.float(), v.float(), key_lengths=klen)
    assert orc.rel_err(results[0][0], want) < tol
    # what the node keeps: the raw inputs, V, the mask, the denominator and the result
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    with ftb.mode(mode):
        y = att(qd, kd, vd, *masks)
    assert type(y.grad_fn).__name__ == "_FusedElu1CausalLinearBackward"
    assert len(y.grad_fn.saved_tensors) == 6


@pytest.mark.parametrize("n_dims,shape", [(256, (2, 300, 3, 64)), (128, (1, 129, 2, 64)), (256, (5, 64))])
def test_native_favor_feature_map(golden, n_dims, shape):
    """Favor's positive random features, forward and backward one pass each on the tensor cores
    (tensor-core mode), against the fp64 restatement of the reference's formula and its gradient; in the fp32 mode the
    reference's torch formulation runs and matches to fp32 accuracy."""
    import fast_transformers_b200 as ftb
    from fast_transformers_b200 import _native
    torch.manual_seed(11)
    fm = Favor(64, n_dims=n_dims, redraw=10 ** 9).cuda()
    fm.new_feature_map("cuda")
    x = (torch.randn(*shape) * 0.6)
    w = torch.rand(*shape[:-1], n_dims)
    omega = fm.omega.double().cpu()
    xd = x.double().requires_grad_(True)
    want = orc.favor_features(xd, omega)
    (want * w.double()).sum().backward()
    for mode, tol in (("mma", 2e-2), ("fp32", 1e-5)):
        xg = x.cuda().requires_grad_(True)
        n0 = _native.lib().ftb_launch_count()
        with ftb.mode(mode):
            phi = fm(xg)
        launched = _native.lib().ftb_launch_count() - n0
        assert launched == (1 if mode == "mma" else 0)
        n0 = _native.lib().ftb_launch_count()
        (phi * w.cuda()).sum().backward()
        assert _native.lib().ftb_launch_count() - n0 == (1 if mode == "mma" else 0)   # the native backward
        assert phi.shape == want.shape and torch.all(phi > 0)
        assert orc.rel_err(phi, want) < tol, mode
        assert orc.rel_err(xg.grad, xd.grad) < tol, mode


def test_native_favor_feature_map_against_the_reference(golden):
    """The reference's own Favor output and input gradient (fixture from the unmodified module,
    64-wide inputs, 256 features) against the native pass."""
    import fast_transformers_b200 as ftb
    g = golden("favor64")
    fm = Favor(64, n_dims=256, redraw=10 ** 9).cuda()
    fm.omega.copy_(T(g["omega"]).cuda())
    x = T(g["x"]).cuda().requires_grad_(True)
    with ftb.mode("mma"):
        phi = fm(x)
    (phi * T(g["w"]).cuda()).sum().backward()
    assert orc.rel_err(phi, T(g["phi"])) < 2e-2
    assert orc.rel_err(x.grad, T(g["gx"])) < 2e-2


def test_layer_with_128_wide_fp32_heads_in_tensor_core_mode():
    """fp32 tensors with 128-wide heads in tensor-core mode (the product through the wide scans,
    the denominator through the streaming kernels): the fp64 layer output, and gradients that agree
    with the fp32 mode's."""
    import fast_transformers_b200 as ftb
    g = torch.Generator().manual_seed(128)
    N, L, H, E = 2, 520, 2, 128
    q, k, v, w = (torch.randn(N, L, H, E, generator=g) for _ in range(4))
    klen = torch.tensor([520, 301])
    masks = (TriangularCausalMask(L, device="cuda"), LengthMask(torch.full((N,), L, device="cuda")),
             LengthMask(klen.cuda(), max_len=L))
    att = CausalLinearAttention(E)
    res = {}
    for mode in ("mma", "fp32"):
        qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
        with ftb.mode(mode):
            y = att(qd, kd, vd, *masks)
            (y * w.cuda()).sum().backward()
        res[mode] = (y.detach(), qd.grad, kd.grad, vd.grad)
    assert orc.rel_err(res["mma"][0], orc.layer_forward(q, k, v, key_lengths=klen)) < 2e-2
    for a, b in zip(res["mma"], res["fp32"]):
        assert orc.rel_err(a, b.double()) < 2e-2
