"""Parity of the tensor-core ("mma") mode -- tcgen05 MMAs with TF32 operands for fp32
tensors and bf16 operands for bf16 tensors, fp32 accumulation and state -- against the fp64
oracle.  Tolerance: 2e-2 on max|x - x64| / max|x64| (fp32-mode tests use 1e-5)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import causal_oracle as orc  # noqa: E402
from fast_transformers_b200 import _native, workloads  # noqa: E402
import fast_transformers_b200 as ftb  # noqa: E402
from fast_transformers_b200.causal_product import (  # noqa: E402
    causal_dot_backward_cuda, causal_dot_product, causal_dot_product_cuda, causal_state_sum)

TOL = 2e-2
NAMES = ("out", "gQ", "gK", "gV")


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available()
    yield native_lib
    torch.cuda.synchronize()
    assert native_lib.ftb_device_status(1) == 0, "a kernel recorded a device-side error"


def fwd_bwd(Q, K, V, G):
    q, k, v = (t.cuda().requires_grad_(True) for t in (Q, K, V))
    with ftb.mode("mma"):
        out = causal_dot_product(q, k, v)
        out.backward(G.cuda())
    torch.cuda.synchronize()
    return out.detach(), q.grad, k.grad, v.grad


def oracle(Q, K, V, G):
    Q, K, V, G = (t.float() for t in (Q, K, V, G))
    return (orc.chunked_forward(Q, K, V),) + tuple(orc.chunked_backward(Q, K, V, G))


def check(Q, K, V, G, tol=TOL):
    got, want = fwd_bwd(Q, K, V, G), oracle(Q, K, V, G)
    errs = {}
    for name, a, b in zip(NAMES, got, want):
        assert a.dtype == Q.dtype and a.shape == b.shape
        errs[name] = orc.rel_err(a, b)
        assert errs[name] < tol, "%s: rel err %.3e" % (name, errs[name])
    return got, errs


def test_config1_tf32(golden):
    Q, K, V, G = workloads.make_inputs(1)
    got, errs = check(Q, K, V, G)
    g = golden("product_config1_sample")
    rows = torch.from_numpy(g["rows"])
    for name, a in zip(NAMES, got):
        assert orc.rel_err(a.cpu()[:, :, rows], torch.from_numpy(g[name])) < TOL, name
    # TF32 keeps 10 mantissa bits: the error should sit well inside the bound
    assert max(errs.values()) < 5e-3


@pytest.mark.parametrize("L", [1, 100, 128, 129, 1000, 2304])
def test_ragged_lengths_tf32(L):
    g = torch.Generator().manual_seed(L)
    Q, K, V, G = (torch.randn(2, 3, L, 64, generator=g) for _ in range(4))
    check(Q, K, V, G)


def test_many_heads_and_segments_tf32():
    Q, K, V, G = workloads.make_inputs(2, scale_N=2, scale_L=2048)
    check(Q, K, V, G)


def test_config4_recipe_bf16_reduced():
    """bf16 I/O, D = M = 128, fp32 state: config 4's recipe at H4, L8192."""
    Q, K, V, G = workloads.make_inputs(4, scale_L=8192, scale_H=4)
    assert Q.dtype == torch.bfloat16
    check(Q, K, V, G)


@pytest.mark.parametrize("L", [77, 640])
def test_bf16_ragged(L):
    g = torch.Generator().manual_seed(L)
    Q, K, V, G = (torch.randn(1, 2, L, 128, generator=g).to(torch.bfloat16) for _ in range(4))
    check(Q, K, V, G)


@pytest.mark.parametrize("L", [77, 640, 2304])
def test_bf16_head_dimension_64(L):
    """bf16 tensors with D = M = 64 (the `<bf16, 64, 64>` instantiation: 64-lane state
    accumulators, one 128-byte block per row)."""
    g = torch.Generator().manual_seed(64 + L)
    Q, K, V, G = (torch.randn(2, 3, L, 64, generator=g).to(torch.bfloat16) for _ in range(4))
    check(Q, K, V, G)


def test_bf16_head_dimension_64_many_heads_long():
    g = torch.Generator().manual_seed(65)
    H, L = 40, 4096
    Q, K, V, G = (torch.rand(2, H, L, 64, generator=g).to(torch.bfloat16) for _ in range(4))
    got = fwd_bwd(Q, K, V, G)
    want = oracle(*(t[1:, 7:9] for t in (Q, K, V, G)))
    for name, a, b in zip(NAMES, got, want):
        assert orc.rel_err(a[1:, 7:9], b) < TOL, name


def test_bf16_long_segments():
    """Enough (batch, head) pairs that a segment is a whole sequence of 10 chunks (config 4 runs
    228 chunks per segment): the barrier phases wrap several times.  Checked on four heads."""
    g = torch.Generator().manual_seed(5)
    H, L = 148, 1280
    Q, K, V, G = (torch.rand(1, H, L, 128, generator=g).to(torch.bfloat16) for _ in range(4))
    got = fwd_bwd(Q, K, V, G)
    heads = [0, 1, 77, 147]
    want = oracle(*(t[:, heads] for t in (Q, K, V, G)))
    for name, a, b in zip(NAMES, got, want):
        assert orc.rel_err(a[:, heads], b) < TOL, name


def test_tf32_long_segments_three_scans_in_one_grid():
    """128 heads -> one segment of 24 chunks per head, no state pass: the backward is one grid of
    three interleaved scans."""
    g = torch.Generator().manual_seed(6)
    H, L = 128, 3072
    Q, K, V, G = (torch.rand(1, H, L, 64, generator=g) for _ in range(4))
    got = fwd_bwd(Q, K, V, G)
    heads = [0, 63, 127]
    want = oracle(*(t[:, heads] for t in (Q, K, V, G)))
    for name, a, b in zip(NAMES, got, want):
        assert orc.rel_err(a[:, heads], b) < TOL, name


@pytest.mark.parametrize("L", [384, 640, 1152])
def test_short_sequences_many_heads_tf32(L):
    """64 (batch, head) pairs and a few chunks: segments of one or two chunks, an odd number of
    chunks (the last segment is shorter, a sub-segment of the state sweep may be empty)."""
    g = torch.Generator().manual_seed(L)
    Q, K, V, G = (torch.rand(8, 8, L, 64, generator=g) for _ in range(4))
    got = fwd_bwd(Q, K, V, G)
    want = oracle(*(t[:2, 3:5] for t in (Q, K, V, G)))
    for name, a, b in zip(NAMES, got, want):
        assert orc.rel_err(a[:2, 3:5], b) < TOL, name


def test_config5_favor_features_tf32_reduced():
    """D = 256 Favor features, M = 64 (config 5's recipe at N1 H2 L2048): the tensor-core mode
    runs it as four 64-wide feature blocks."""
    Q, K, V, G = workloads.make_inputs(5, scale_N=1, scale_H=2, scale_L=2048)
    assert Q.shape[3] == 256 and V.shape[3] == 64
    check(Q, K, V, G)


def test_nlhd_storage_views_tf32():
    """(N, L, H, D) storage viewed as (N, H, L, D): the head stride is below the row stride."""
    g = torch.Generator().manual_seed(21)
    N, L, H, D = 2, 700, 3, 64
    Qs, Ks, Vs, Gs = (torch.randn(N, L, H, D, generator=g) for _ in range(4))
    q, k, v = (t.cuda().permute(0, 2, 1, 3).requires_grad_(True) for t in (Qs, Ks, Vs))
    assert not q.is_contiguous()
    with ftb.mode("mma"):
        out = causal_dot_product(q, k, v)
        out.backward(Gs.cuda().permute(0, 2, 1, 3))
    want = oracle(*(t.permute(0, 2, 1, 3) for t in (Qs, Ks, Vs, Gs)))
    for name, a, b in zip(NAMES, (out, q.grad, k.grad, v.grad), want):
        assert orc.rel_err(a, b) < TOL, name


def test_states_split_sequence_tf32():
    g = torch.Generator().manual_seed(22)
    N, H, L, D = 1, 2, 1536, 64
    Q, K, V, G = (torch.rand(N, H, L, D, generator=g) for _ in range(4))
    Qd, Kd, Vd, Gd = (t.cuda() for t in (Q, K, V, G))
    h = 640
    want_o = orc.chunked_forward(Q, K, V)
    want_g = orc.chunked_backward(Q, K, V, G)
    S0 = causal_state_sum(Kd[:, :, :h], Vd[:, :, :h], mode="mma")
    assert orc.rel_err(S0, orc.local_states(None, K[:, :, :h], V[:, :, :h])) < TOL
    o1 = torch.empty(N, H, h, D, device="cuda")
    o2 = torch.empty(N, H, L - h, D, device="cuda")
    fin = torch.empty(N, H, D, D, device="cuda")
    causal_dot_product_cuda(Qd[:, :, :h], Kd[:, :, :h], Vd[:, :, :h], o1, "mma", final_state=fin)
    assert orc.rel_err(fin, S0) < 1e-5
    causal_dot_product_cuda(Qd[:, :, h:], Kd[:, :, h:], Vd[:, :, h:], o2, "mma", initial_state=fin)
    assert orc.rel_err(torch.cat([o1, o2], 2), want_o) < TOL
    R1 = causal_state_sum(Qd[:, :, h:], Gd[:, :, h:], mode="mma")
    g1 = [torch.empty(N, H, h, D, device="cuda") for _ in range(3)]
    g2 = [torch.empty(N, H, L - h, D, device="cuda") for _ in range(3)]
    causal_dot_backward_cuda(Qd[:, :, :h], Kd[:, :, :h], Vd[:, :, :h], Gd[:, :, :h], *g1, "mma",
                             initial_grad_state=R1)
    causal_dot_backward_cuda(Qd[:, :, h:], Kd[:, :, h:], Vd[:, :, h:], Gd[:, :, h:], *g2, "mma",
                             initial_state=fin)
    for a, b, c in zip(g1, g2, want_g):
        assert orc.rel_err(torch.cat([a, b], 2), c) < TOL


def test_forward_workspace_reuse_is_bitwise_equal_to_recompute():
    Q, K, V, G = workloads.make_inputs(1)
    Qd, Kd, Vd, Gd = (t.cuda() for t in (Q, K, V, G))
    out = torch.empty_like(Vd)
    kept = []
    causal_dot_product_cuda(Qd, Kd, Vd, out, "mma", keep_workspace=kept)
    a = [torch.empty_like(t) for t in (Qd, Kd, Vd)]
    b = [torch.empty_like(t) for t in (Qd, Kd, Vd)]
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *a, "mma", forward_workspace=kept[0])
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *b, "mma")
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("mode", ["mma", "fp32"])
def test_gradients_asked_for_separately_equal_the_joint_call(mode):
    """A gradient buffer given as None is skipped; what is computed is bitwise what the call for
    all three computes (config 1: two segments per head, so both state sweeps are involved)."""
    Q, K, V, G = (t.cuda() for t in workloads.make_inputs(1))
    full = [torch.empty_like(t) for t in (Q, K, V)]
    causal_dot_backward_cuda(Q, K, V, G, *full, mode)
    gq = torch.full_like(Q, float("nan"))
    gk, gv = torch.full_like(K, float("nan")), torch.full_like(V, float("nan"))
    causal_dot_backward_cuda(Q, K, V, G, gq, None, None, mode)
    causal_dot_backward_cuda(Q, K, V, G, None, gk, gv, mode)
    for a, b in zip(full, (gq, gk, gv)):
        assert torch.equal(a, b)
    only_v = torch.full_like(V, float("nan"))
    causal_dot_backward_cuda(Q, K, V, G, None, None, only_v, mode)
    assert torch.equal(only_v, full[2])
    with pytest.raises(RuntimeError):
        causal_dot_backward_cuda(Q, K, V, G, None, None, None, mode)


def test_determinism_tf32():
    Q, K, V, G = workloads.make_inputs(1)
    a, b = fwd_bwd(Q, K, V, G), fwd_bwd(Q, K, V, G)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_unsupported_shape_and_alignment_errors():
    x = torch.rand(1, 1, 256, 32, device="cuda")
    out = torch.empty_like(x)
    with pytest.raises(_native.NativeError) as e:
        causal_dot_product_cuda(x, x, x, out, "mma")
    assert e.value.status == _native.ERR_UNSUPPORTED
    # a view that starts 4 bytes into a row: TMA needs 16-byte aligned bases
    big = torch.rand(1, 1, 256, 80, device="cuda")
    mis = big[..., 1:65]
    out = torch.empty(1, 1, 256, 64, device="cuda")
    with pytest.raises(_native.NativeError) as e:
        causal_dot_product_cuda(mis, mis, mis, out, "mma")
    assert e.value.status == _native.ERR_ALIGNMENT


def test_linearity_config2_full_size_tf32():
    """Full-size config 2: out is linear in V (exactly, scaling by 2 is exact in TF32), the
    first row is (q_0 . k_0) v_0 and the last row is q_L . K^T V."""
    Q, K, V, _ = workloads.make_inputs(2)
    Qd, Kd, Vd = (t.cuda() for t in (Q, K, V))
    with ftb.mode("mma"):
        o1 = causal_dot_product(Qd, Kd, Vd)
        o2 = causal_dot_product(Qd, Kd, 2.0 * Vd)
    assert torch.equal(o2, 2.0 * o1)
    S = K.double().transpose(-1, -2) @ V.double()
    assert orc.rel_err(o1[:, :, -1:], Q[:, :, -1:].double() @ S) < TOL
    first = (Q[:, :, :1].double() * K[:, :, :1].double()).sum(-1, keepdim=True) * V[:, :, :1].double()
    assert orc.rel_err(o1[:, :, :1], first) < TOL


def test_kept_states_are_read_in_the_layout_they_were_written_in():
    """Two (batch, head) pairs, L = 2048: eight segments per pair and two state blocks per segment.
    Whoever wrote the per-segment states -- a forward call that also returns its final state, or
    ``causal_state_sum`` followed by a forward call that reuses its workspace -- the backward call
    given that workspace must read them as they were written (against the oracle, all gradients)."""
    g = torch.Generator().manual_seed(41)
    N, H, L, D = 1, 2, 2048, 64
    Q, K, V, G = (torch.rand(N, H, L, D, generator=g) for _ in range(4))
    Qd, Kd, Vd, Gd = (t.cuda() for t in (Q, K, V, G))
    want = oracle(Q, K, V, G)

    def backward_with(ws):
        grads = [torch.full_like(t, float("nan")) for t in (Qd, Kd, Vd)]
        causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *grads, "mma", forward_workspace=ws)
        return grads

    # (a) forward with final_state, workspace kept, backward reuses it
    out = torch.empty_like(Vd)
    fin = torch.empty(N, H, D, D, device="cuda")
    kept = []
    causal_dot_product_cuda(Qd, Kd, Vd, out, "mma", final_state=fin, keep_workspace=kept)
    assert kept[0] is not None
    for name, a, b in zip(NAMES, [out] + backward_with(kept[0]), want):
        assert orc.rel_err(a, b) < TOL, "(a) " + name
    assert orc.rel_err(fin, orc.local_states(None, K, V)) < TOL
    # (b) causal_state_sum first, forward on its workspace, backward reuses it
    from fast_transformers_b200.causal_product import workspace_bytes
    ws = torch.empty(workspace_bytes(N, H, L, D, D, torch.float32, "mma", want_state=True),
                     dtype=torch.uint8, device="cuda")
    total = causal_state_sum(Kd, Vd, mode="mma", workspace=ws)
    assert orc.rel_err(total, fin) < 1e-5
    out2 = torch.full_like(Vd, float("nan"))
    causal_dot_product_cuda(Qd, Kd, Vd, out2, "mma", workspace=ws, workspace_has_states=True)
    for name, a, b in zip(NAMES, [out2] + backward_with(ws), want):
        assert orc.rel_err(a, b) < TOL, "(b) " + name
    # (c) the plain forward's workspace (no final state)
    kept = []
    out3 = torch.empty_like(Vd)
    causal_dot_product_cuda(Qd, Kd, Vd, out3, "mma", keep_workspace=kept)
    for name, a, b in zip(NAMES, [out3] + backward_with(kept[0]), want):
        assert orc.rel_err(a, b) < TOL, "(c) " + name


@pytest.mark.parametrize("D,L,H", [(192, 900, 3), (128, 1300, 2), (256, 2500, 5), (320, 700, 2), (256, 128, 1),
                                   (128, 40000, 1)])
def test_wide_feature_products_are_summed_by_the_library(D, L, H):
    """D = 64 nb (two to five 64-wide feature blocks), M = 64, fp32, tensor-core mode: one native call
    per direction.  out and grad_V (wide on the query / key side) are summed over the blocks inside
    the tensor cores, up to four blocks per launch (D = 320: a second launch adds the fifth); they
    hold NaN on entry, so the first launch must replace.  grad_Q and grad_K (wide on the output
    side) stream up to four column blocks per launch past scores made once per chunk (D = 320: the
    fifth block through the 64-wide scan).  One long sequence alone is cut into more segments than a
    scan adds up itself (a prefix launch turns the totals into start states).  A skipped gradient is
    honoured; states are refused."""
    g = torch.Generator().manual_seed(D + L)
    N, M = 1, 64
    Q, K = (torch.rand(N, H, L, D, generator=g) * 0.5 for _ in range(2))
    V, G = (torch.randn(N, H, L, M, generator=g) for _ in range(2))
    Qd, Kd, Vd, Gd = (t.cuda() for t in (Q, K, V, G))
    out = torch.full((N, H, L, M), float("nan"), device="cuda")
    kept = []
    n0 = _native.lib().ftb_launch_count()
    causal_dot_product_cuda(Qd, Kd, Vd, out, "mma", keep_workspace=kept)
    grads = [torch.full_like(t, float("nan")) for t in (Qd, Kd, Vd)]
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *grads, "mma", forward_workspace=kept[0])
    assert _native.lib().ftb_launch_count() - n0 >= 3
    want = oracle(Q, K, V, G)
    for name, a, b in zip(NAMES, [out] + grads, want):
        assert orc.rel_err(a, b) < TOL, name
    # without the forward's workspace the backward sweeps (K, V) itself: same result
    grads2 = [torch.full_like(t, float("nan")) for t in (Qd, Kd, Vd)]
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *grads2, "mma")
    for a, b in zip(grads, grads2):
        assert torch.equal(a, b)
    only_v = torch.full_like(Vd, float("nan"))
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, None, None, only_v, "mma")
    assert torch.equal(only_v, grads[2])
    only_q = torch.full_like(Qd, float("nan"))
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, only_q, None, None, "mma")
    assert orc.rel_err(only_q, want[1]) < TOL
    with pytest.raises(_native.NativeError) as e:
        causal_dot_product_cuda(Qd, Kd, Vd, out, "mma", initial_state=torch.zeros(N, H, D, M, device="cuda"))
    assert e.value.status == _native.ERR_UNSUPPORTED


@pytest.mark.parametrize("dtype,D", [(torch.float32, 64), (torch.bfloat16, 128), (torch.bfloat16, 64)])
def test_normaliser_applied_in_the_epilogue(dtype, D):
    """``row_den``: row i of the product is divided by den[i] + eps as the scan stores it
    (``ftb_causal_dot_product_normalised``), den given as an (N, H, L) view of (N, L, H) storage.
    For fp32 the result is, bit for bit, the plain product times 1 / (den + eps)."""
    g = torch.Generator().manual_seed(D)
    N, H, L, eps = 2, 3, 1100, 1e-6
    Q, K = (torch.rand(N, H, L, D, generator=g).to(dtype) for _ in range(2))
    V = torch.randn(N, H, L, D, generator=g).to(dtype)
    den = (torch.rand(N, L, H, generator=g) * 50 + 0.5).cuda().permute(0, 2, 1)
    Qd, Kd, Vd = Q.cuda(), K.cuda(), V.cuda()
    plain, scaled = torch.empty_like(Vd), torch.full_like(Vd, float("nan"))
    causal_dot_product_cuda(Qd, Kd, Vd, plain, "mma")
    causal_dot_product_cuda(Qd, Kd, Vd, scaled, "mma", row_den=den, eps=eps)
    z = 1 / (den + eps)
    if dtype == torch.float32:
        assert torch.equal(scaled, plain * z[..., None])
    want = orc.chunked_forward(Q.float(), K.float(), V.float()) * z.cpu().double()[..., None]
    assert orc.rel_err(scaled, want) < TOL
    with pytest.raises(_native.NativeError) as e:       # the fp32 kernels have no such epilogue
        causal_dot_product_cuda(Qd.float(), Kd.float(), Vd.float(), plain.float(), "fp32", row_den=den, eps=eps)
    assert e.value.status == _native.ERR_UNSUPPORTED
    with pytest.raises(RuntimeError):
        causal_dot_product_cuda(Qd, Kd, Vd, scaled, "mma", row_den=den.double(), eps=eps)


@pytest.mark.parametrize("D,M,L,H", [(64, 128, 700, 3), (128, 128, 1500, 2), (192, 128, 900, 2), (128, 192, 640, 3),
                                     (320, 128, 400, 1), (64, 320, 300, 2)])
def test_fp32_widths_that_are_multiples_of_64(D, M, L, H):
    """fp32 tensors in tensor-core mode with any query / value widths that are multiples of 64: the
    sums over 64-wide feature blocks (of the queries for out and grad_V, of the values for grad_Q and
    grad_K) are taken inside the tensor cores, one launch per 64 columns of the other side and per
    group of four blocks.  Outputs hold NaN on entry; with and without the forward's workspace."""
    g = torch.Generator().manual_seed(D * 7 + M)
    N = 2
    Q, K = (torch.rand(N, H, L, D, generator=g) * 0.5 for _ in range(2))
    V, G = (torch.randn(N, H, L, M, generator=g) for _ in range(2))
    Qd, Kd, Vd, Gd = (t.cuda() for t in (Q, K, V, G))
    out = torch.full((N, H, L, M), float("nan"), device="cuda")
    kept = []
    causal_dot_product_cuda(Qd, Kd, Vd, out, "mma", keep_workspace=kept)
    grads = [torch.full_like(t, float("nan")) for t in (Qd, Kd, Vd)]
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *grads, "mma", forward_workspace=kept[0])
    want = oracle(Q, K, V, G)
    for name, a, b in zip(NAMES, [out] + grads, want):
        assert orc.rel_err(a, b) < TOL, name
    again = [torch.full_like(t, float("nan")) for t in (Qd, Kd, Vd)]
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, *again, "mma")
    for a, b in zip(grads, again):
        assert torch.equal(a, b)
    # through autograd as well
    q, k, v = (t.clone().requires_grad_(True) for t in (Qd, Kd, Vd))
    with ftb.mode("mma"):
        causal_dot_product(q, k, v).backward(Gd)
    for a, b in zip(grads, (q.grad, k.grad, v.grad)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("D,M", workloads.WIDE_GOLDEN_SHAPES)
def test_wide_shapes_against_the_reference(golden, D, M):
    """The reference's own outputs and gradients for widths that are multiples of 64 above 64
    (fixture from its unmodified CPU kernel; sampled rows): tensor-core mode within 2e-2, fp32 mode
    within 1e-5."""
    g = golden("product_wide")
    Q, K, V, G = workloads.wide_golden_inputs(D, M)
    rows = workloads.WIDE_GOLDEN_ROWS
    for mode, tol in (("mma", TOL), ("fp32", 1e-5)):
        q, k, v = (t.cuda().requires_grad_(True) for t in (Q, K, V))
        with ftb.mode(mode):
            out = causal_dot_product(q, k, v)
            out.backward(G.cuda())
        for name, a in zip(NAMES, (out, q.grad, k.grad, v.grad)):
            ref = torch.from_numpy(g["%s_%d_%d" % (name, D, M)])
            assert orc.rel_err(a.detach().cpu()[:, :, rows], ref) < tol, (mode, name)
