"""The unmasked (non-causal) form on the GPU: one fixed state applied to every position
(``ftb_linear_apply_state``), the product ``Q (K^T V)`` and its gradients, the ``LinearAttention``
layer and ``RecurrentCrossLinearAttention`` against the reference's outputs (golden fixtures from
the unmodified reference modules) and the fp64 oracle.  Tolerances as everywhere: 1e-5 in the fp32
mode, 2e-2 in the tensor-core mode, on max|x - x64| / max|x64|."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import causal_oracle as orc  # noqa: E402
import fast_transformers_b200 as ftb  # noqa: E402
from fast_transformers_b200 import _native  # noqa: E402
from fast_transformers_b200.attention import LinearAttention  # noqa: E402
from fast_transformers_b200.attention_registry import (AttentionRegistry,  # noqa: E402
                                                       RecurrentCrossAttentionRegistry)
from fast_transformers_b200.causal_product.linear_product import (linear_apply_state,  # noqa: E402
                                                                  linear_dot_product)
from fast_transformers_b200.masking import FullMask, LengthMask  # noqa: E402
from fast_transformers_b200.recurrent.attention import RecurrentCrossLinearAttention  # noqa: E402

TOL = {"fp32": 1e-5, "mma": 2e-2}


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available()
    yield native_lib
    torch.cuda.synchronize()
    assert native_lib.ftb_device_status(1) == 0


def T(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("mode,dtype,Da,Dc,L", [
    ("fp32", torch.float32, 64, 64, 300), ("fp32", torch.float32, 37, 90, 129),
    ("fp32", torch.bfloat16, 32, 48, 65), ("fp32", torch.float32, 256, 64, 500),
    ("mma", torch.float32, 64, 64, 1000), ("mma", torch.float32, 64, 64, 128),
    ("mma", torch.float32, 64, 128, 333), ("mma", torch.bfloat16, 128, 128, 700),
    ("mma", torch.bfloat16, 64, 64, 450)])
@pytest.mark.parametrize("transposed", [False, True])
def test_apply_state_against_fp64(mode, dtype, Da, Dc, L, transposed):
    g = torch.Generator().manual_seed(Da + Dc + L)
    N, H = 2, 3
    a = torch.randn(N, H, L, Da, generator=g).to(dtype)
    S = torch.randn(N, H, Da, Dc, generator=g)
    stored = S.transpose(2, 3).contiguous() if transposed else S
    out = linear_apply_state(a.cuda(), stored.cuda(), mode=mode, transposed=transposed)
    assert out.shape == (N, H, L, Dc) and out.dtype == dtype
    tol = TOL[mode] if dtype == torch.float32 else 2e-2     # bf16 output rounding
    assert orc.rel_err(out, a.double() @ S.double()) < tol


def test_apply_state_reads_and_writes_nlhd_storage():
    """(N, L, H, D) storage viewed as (N, H, L, D), in and out, tensor-core mode."""
    g = torch.Generator().manual_seed(5)
    N, L, H, D = 2, 260, 3, 64
    a = torch.randn(N, L, H, D, generator=g)
    S = torch.randn(N, H, D, D, generator=g)
    out_store = torch.full((N, L, H, D), float("nan"), device="cuda")
    linear_apply_state(a.cuda().permute(0, 2, 1, 3), S.cuda(), out_store.permute(0, 2, 1, 3), mode="mma")
    want = a.permute(0, 2, 1, 3).double() @ S.double()
    assert orc.rel_err(out_store.permute(0, 2, 1, 3), want) < TOL["mma"]


def test_apply_state_status_codes(native_lib):
    a = torch.zeros(1, 1, 128, 32, device="cuda")
    S = torch.zeros(1, 1, 32, 32, device="cuda")
    with pytest.raises(_native.NativeError) as e:
        linear_apply_state(a, S, mode="mma")          # no tensor-core kernel for D = 32
    assert e.value.status == _native.ERR_UNSUPPORTED
    with pytest.raises(RuntimeError):
        linear_apply_state(a, torch.zeros(1, 1, 16, 32, device="cuda"), mode="fp32")
    assert linear_apply_state(a[:, :, :0], S, mode="fp32").shape == (1, 1, 0, 32)


@pytest.mark.parametrize("mode,dtype,D,M", [("fp32", torch.float32, 40, 24), ("fp32", torch.float32, 64, 64),
                                            ("mma", torch.float32, 64, 64), ("mma", torch.bfloat16, 128, 128)])
def test_unmasked_product_and_gradients(mode, dtype, D, M):
    """Q (K^T V) with queries and keys of different lengths, all three gradients."""
    g = torch.Generator().manual_seed(D + M)
    N, H, L, S = 2, 3, 700, 900
    Q = (torch.rand(N, H, L, D, generator=g) * 0.5).to(dtype)
    K = (torch.rand(N, H, S, D, generator=g) * 0.5).to(dtype)
    V = torch.randn(N, H, S, M, generator=g).to(dtype)
    G = torch.randn(N, H, L, M, generator=g).to(dtype)
    q, k, v = (t.cuda().requires_grad_(True) for t in (Q, K, V))
    with ftb.mode(mode):
        out = linear_dot_product(q, k, v)
        out.backward(G.cuda())
    want = orc.linear_product(Q.float(), K.float(), V.float(), G.float())
    tol = TOL[mode] if dtype == torch.float32 else 2e-2
    for name, a, b in zip(("out", "gQ", "gK", "gV"), (out, q.grad, k.grad, v.grad), want):
        assert a.dtype == dtype and a.shape == b.shape
        assert orc.rel_err(a, b) < tol, name


def test_layer_matches_reference(golden):
    g = golden("linear")
    q, k, v, w = (T(g[n]).cuda() for n in "qkvw")
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    N, L = q.shape[:2]
    S = k.shape[1]
    klm = LengthMask(T(g["klen"]).cuda(), max_len=S)
    att = LinearAttention(q.shape[3])
    y = att(q, k, v, FullMask(L, S, device="cuda"), LengthMask(torch.full((N,), L, device="cuda")), klm)
    assert y.is_contiguous() and y.shape == (N, L, q.shape[2], v.shape[3])
    assert (y.cpu() - T(g["y"])).abs().max() < 1e-5
    assert orc.rel_err(y, orc.linear_layer_forward(q, k, v, key_lengths=T(g["klen"]))) < 1e-5
    (y * w).sum().backward()
    for n, t in (("gq", q), ("gk", k), ("gv", v)):
        assert orc.rel_err(t.grad, T(g[n])) < 1e-5, n
    with pytest.raises(RuntimeError):        # a mask that is not all ones is refused, as in the reference
        att(q, k, v, FullMask(torch.tril(torch.ones(L, S)).bool().cuda()),
            LengthMask(torch.full((N,), L, device="cuda")), klm)


def test_layer_tensor_core_mode_against_oracle():
    g = torch.Generator().manual_seed(9)
    N, L, S, H, E = 2, 400, 520, 4, 64
    q, k, v = (torch.randn(N, n, H, E, generator=g) for n in (L, S, S))
    klen = torch.tensor([520, 333])
    att = LinearAttention(E)
    with ftb.mode("mma"):
        y = att(q.cuda(), k.cuda(), v.cuda(), FullMask(L, S, device="cuda"),
                LengthMask(torch.full((N,), L, device="cuda")), LengthMask(klen.cuda(), max_len=S))
    assert orc.rel_err(y, orc.linear_layer_forward(q, k, v, key_lengths=klen)) < TOL["mma"]


def test_recurrent_cross_attention_matches_reference(golden):
    g = golden("linear")
    q, k, v = (T(g[n]).cuda() for n in "qkv")
    L, S = q.shape[1], k.shape[1]
    klm = LengthMask(T(g["klen"]).cuda(), max_len=S)
    rec = RecurrentCrossLinearAttention(q.shape[3]).eval()
    with torch.no_grad():
        state, ys = None, []
        for i in range(L):
            y, state = rec(q[:, i], k, v, klm, state)
            ys.append(y)
    assert (torch.stack(ys, 1).cpu() - T(g["step_y"])).abs().max() < 1e-5
    # the state has the reference's shapes: S (N, H, M, D), z (N, H, D)
    assert state[0].shape == g["state_S"].shape and state[1].shape == g["state_z"].shape
    assert orc.rel_err(state[0], T(g["state_S"])) < 1e-5
    assert orc.rel_err(state[1], T(g["state_z"])) < 1e-5
    # a state handed in from outside (a contiguous (N, H, M, D) tensor, as the reference makes it)
    with torch.no_grad():
        y2, _ = rec(q[:, 0], k, v, klm, [T(g["state_S"]).cuda(), T(g["state_z"]).cuda()])
    assert (y2.cpu() - T(g["step_y"])[:, 0]).abs().max() < 1e-5
    with pytest.raises(RuntimeError):
        rec(q[:, 0].clone().requires_grad_(True), k, v, klm)


def test_registry_entries():
    cls, params = AttentionRegistry["linear"]
    assert cls is LinearAttention and params == ["query_dimensions", "feature_map", "event_dispatcher"]
    cls, params = RecurrentCrossAttentionRegistry["linear"]
    assert cls is RecurrentCrossLinearAttention
    assert params == ["query_dimensions", "feature_map", "event_dispatcher"]
