"""The split-operand tensor-core mode (``"tf32x3"``): fp32 operands as a TF32-exact high part plus a
low part, three products per product, fp32 accumulation -- the accuracy tier of the fp32 CUDA-core
kernels (1e-5 on max|x - x64| / max|x64| against the fp64 oracle) on the tensor cores.  Native
kernels for fp32 tensors with D = M = 64; the Python layer runs every other shape as ``"fp32"``."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import causal_oracle as orc  # noqa: E402
from fast_transformers_b200 import _native, workloads  # noqa: E402
import fast_transformers_b200 as ftb  # noqa: E402
from fast_transformers_b200.attention import CausalLinearAttention  # noqa: E402
from fast_transformers_b200.causal_product import (  # noqa: E402
    causal_dot_backward_cuda, causal_dot_product, causal_dot_product_cuda, workspace_bytes)
from fast_transformers_b200.masking import LengthMask, TriangularCausalMask  # noqa: E402

TOL = 1e-5
NAMES = ("out", "gQ", "gK", "gV")


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available()
    yield native_lib
    torch.cuda.synchronize()
    assert native_lib.ftb_device_status(1) == 0, "a kernel recorded a device-side error"


def oracle(Q, K, V, G):
    return (orc.chunked_forward(Q, K, V),) + tuple(orc.chunked_backward(Q, K, V, G))


def run(Q, K, V, G, mode="tf32x3"):
    q, k, v = (t.cuda().requires_grad_(True) for t in (Q, K, V))
    with ftb.mode(mode):
        out = causal_dot_product(q, k, v)
        out.backward(G.cuda())
    torch.cuda.synchronize()
    return out.detach(), q.grad, k.grad, v.grad


def check(Q, K, V, G, tol=TOL):
    n0 = _native.lib().ftb_launch_count()
    got, want = run(Q, K, V, G), oracle(Q, K, V, G)
    assert _native.lib().ftb_launch_count() > n0
    errs = {}
    for name, a, b in zip(NAMES, got, want):
        assert a.dtype == Q.dtype and a.shape == b.shape
        errs[name] = orc.rel_err(a, b)
        assert errs[name] < tol, "%s: rel err %.3e" % (name, errs[name])
    return got, errs


def test_config1(golden):
    """The reference's own CPU-runnable case, against the oracle and the reference's outputs."""
    Q, K, V, G = workloads.make_inputs(1)
    got, errs = check(Q, K, V, G)
    g = golden("product_config1_sample")
    rows = torch.from_numpy(g["rows"])
    for name, a in zip(NAMES, got):
        assert orc.rel_err(a.cpu()[:, :, rows], torch.from_numpy(g[name])) < TOL, name
    # the three-product split leaves ~2^-21 per product: well inside the bound
    print("tf32x3 config 1 errors", errs)
    assert max(errs.values()) < 5e-6


@pytest.mark.parametrize("L", [1, 100, 128, 129, 1000, 2304])
def test_ragged_lengths_signed_inputs(L):
    g = torch.Generator().manual_seed(L)
    Q, K, V, G = (torch.randn(2, 3, L, 64, generator=g) for _ in range(4))
    check(Q, K, V, G)


@pytest.mark.parametrize("N,H,L", [(1, 1, 4096), (2, 2, 8192), (1, 40, 3000), (3, 50, 1100), (1, 2, 40000)])
def test_segment_counts(N, H, L):
    """One pair split into many segments (raw totals added up by the scan; past 16 segments a prefix
    launch), many pairs with one segment each, and the cases in between."""
    g = torch.Generator().manual_seed(N * 1000 + L)
    Q, K = (torch.nn.functional.elu(torch.randn(N, H, L, 64, generator=g)) + 1 for _ in range(2))
    V, G = (torch.randn(N, H, L, 64, generator=g) for _ in range(2))
    check(Q, K, V, G)


def test_matches_the_fp32_kernels_closely():
    """Both 1e-5-tier paths on one input: they agree with each other far inside the tolerance."""
    Q, K, V, G = workloads.make_inputs(2, scale_N=1, scale_L=2048)
    a, b = run(Q, K, V, G, "tf32x3"), run(Q, K, V, G, "fp32")
    for name, x, y in zip(NAMES, a, b):
        assert orc.rel_err(x, y.double()) < 5e-6, name


def test_strided_storage_and_prefilled_outputs():
    """(N, L, H, D) storage viewed as (N, H, L, D); outputs hold NaN on entry; the backward with and
    without the forward's workspace, and with one gradient skipped."""
    g = torch.Generator().manual_seed(7)
    N, L, H = 2, 1500, 3
    Q, K = (torch.rand(N, L, H, 64, generator=g) for _ in range(2))
    V, G = (torch.randn(N, L, H, 64, generator=g) for _ in range(2))
    Qd, Kd, Vd, Gd = (t.cuda().permute(0, 2, 1, 3) for t in (Q, K, V, G))
    want = oracle(*(t.permute(0, 2, 1, 3) for t in (Q, K, V, G)))
    out = torch.full((N, L, H, 64), float("nan"), device="cuda").permute(0, 2, 1, 3)
    kept = []
    causal_dot_product_cuda(Qd, Kd, Vd, out, "tf32x3", keep_workspace=kept)
    grads = [torch.full((N, L, H, 64), float("nan"), device="cuda").permute(0, 2, 1, 3) for _ in range(3)]
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *grads, "tf32x3", forward_workspace=kept[0])
    for name, a, b in zip(NAMES, [out] + grads, want):
        assert orc.rel_err(a, b) < TOL, name
    again = [torch.full_like(t, float("nan")) for t in grads]
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *again, "tf32x3")
    for a, b in zip(grads, again):
        assert torch.equal(a, b)
    only_k = torch.full_like(grads[1], float("nan"))
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, None, only_k, None, "tf32x3")
    assert torch.equal(only_k, grads[1])


def test_native_entry_refuses_other_shapes_and_python_runs_them_as_fp32(native_lib):
    g = torch.Generator().manual_seed(3)
    Q, K, V, G = (torch.randn(1, 2, 300, 32, generator=g) for _ in range(4))
    q, k, v = (t.cuda() for t in (Q, K, V))
    out = torch.empty_like(v)
    import ctypes
    st = native_lib.ftb_causal_dot_product(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), ctypes.c_void_p(v.data_ptr()),
        ctypes.c_void_p(out.data_ptr()), 1, 2, 300, 32, 32, _native.strides3(q), _native.strides3(k),
        _native.strides3(v), _native.strides3(out), 0, _native.MODE_MMA_X3, None, None, 0, None, 0, None)
    assert st == _native.ERR_UNSUPPORTED
    assert workspace_bytes(1, 2, 300, 32, 32, torch.float32, "tf32x3") == \
        workspace_bytes(1, 2, 300, 32, 32, torch.float32, "fp32")
    got, want = run(Q, K, V, G), oracle(Q, K, V, G)       # D = 32: the fp32 kernels, same tier
    for name, a, b in zip(NAMES, got, want):
        assert orc.rel_err(a, b) < TOL, name
    # a state makes the product an fp32-kernel call too
    S0 = torch.randn(1, 2, 64, 64, generator=g)
    Q, K, V = (torch.randn(1, 2, 200, 64, generator=g) for _ in range(3))
    out = torch.empty(1, 2, 200, 64, device="cuda")
    causal_dot_product_cuda(Q.cuda(), K.cuda(), V.cuda(), out, "tf32x3", initial_state=S0.cuda())
    assert orc.rel_err(out, orc.chunked_forward(Q, K, V, initial_state=S0)) < TOL


def test_layer_in_split_operand_mode():
    """CausalLinearAttention (64-wide heads) with the mode set: the fp64 layer output, and the
    gradients of the fp32 mode."""
    g = torch.Generator().manual_seed(41)
    N, L, H, E = 2, 900, 3, 64
    q, k, v, w = (torch.randn(N, L, H, E, generator=g) for _ in range(4))
    klen = torch.tensor([900, 517])
    masks = (TriangularCausalMask(L, device="cuda"), LengthMask(torch.full((N,), L, device="cuda")),
             LengthMask(klen.cuda(), max_len=L))
    att = CausalLinearAttention(E)
    res = {}
    for mode in ("tf32x3", "fp32"):
        qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
        n0 = _native.lib().ftb_launch_count()
        with ftb.mode(mode):
            y = att(qd, kd, vd, *masks)
            (y * w.cuda()).sum().backward()
        assert _native.lib().ftb_launch_count() > n0
        res[mode] = (y.detach(), qd.grad, kd.grad, vd.grad)
    assert orc.rel_err(res["tf32x3"][0], orc.layer_forward(q, k, v, key_lengths=klen)) < TOL
    for name, a, b in zip(NAMES, res["tf32x3"], res["fp32"]):
        assert orc.rel_err(a, b.double()) < TOL, name
