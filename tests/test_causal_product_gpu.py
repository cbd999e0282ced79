"""Parity of the CUDA kernels (through the C ABI) against the CPU oracle.

Metric: max|x - x64| / max|x64| per tensor (``oracle.causal_oracle.rel_err``).
Tolerances: 1e-5 in the fp32 mode, 2e-2 in the tensor-core ("mma") mode.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import causal_oracle as orc  # noqa: E402
from fast_transformers_b200 import workloads  # noqa: E402
import fast_transformers_b200 as ftb  # noqa: E402
from fast_transformers_b200.causal_product import (  # noqa: E402
    CausalDotProduct, causal_dot_backward_cuda, causal_dot_product, causal_dot_product_cuda,
    causal_state_sum)

TOL = {"fp32": 1e-5, "mma": 2e-2}


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return native_lib


def dev(*ts):
    return [t.cuda() for t in ts]


def run_fwd_bwd(Q, K, V, G, mode):
    Qd, Kd, Vd, Gd = dev(Q, K, V, G)
    Qd.requires_grad_(True), Kd.requires_grad_(True), Vd.requires_grad_(True)
    with ftb.mode(mode):
        out = causal_dot_product(Qd, Kd, Vd)
        out.backward(Gd)
    torch.cuda.synchronize()
    return out.detach(), Qd.grad, Kd.grad, Vd.grad


def check_against_oracle(Q, K, V, G, mode, chunked=False, tol=None):
    tol = tol or TOL[mode]
    got = run_fwd_bwd(Q, K, V, G, mode)
    Qf, Kf, Vf, Gf = (t.float() for t in (Q, K, V, G))
    if chunked:
        want = (orc.chunked_forward(Qf, Kf, Vf),) + tuple(orc.chunked_backward(Qf, Kf, Vf, Gf))
    else:
        want = (orc.dense_forward(Qf, Kf, Vf),) + tuple(orc.dense_backward(Qf, Kf, Vf, Gf))
    for name, a, b in zip(("out", "gQ", "gK", "gV"), got, want):
        assert a.dtype == Q.dtype and a.shape == b.shape
        err = orc.rel_err(a, b)
        assert err < tol, "%s: rel err %.3e (mode %s)" % (name, err, mode)
    return got


def test_golden_small_fp32(golden):
    g = golden("product_small")
    Q, K, V, G = (torch.from_numpy(g[k]) for k in "QKVG")
    got = run_fwd_bwd(Q, K, V, G, "fp32")
    for name, a in zip(("out", "gQ", "gK", "gV"), got):
        ref = torch.from_numpy(g[name])
        # criterion of the reference's tests (test_causal_product_gpu.py:62,82-84)
        assert orc.max_relative_error(ref, a) < 1e-5, name


def test_config1_fp32_vs_oracle_and_reference_sample(golden):
    Q, K, V, G = workloads.make_inputs(1)
    got = check_against_oracle(Q, K, V, G, "fp32", chunked=True)
    g = golden("product_config1_sample")
    rows = torch.from_numpy(g["rows"])
    for name, a in zip(("out", "gQ", "gK", "gV"), got):
        assert orc.rel_err(a.cpu()[:, :, rows], torch.from_numpy(g[name])) < 2e-6, name


@pytest.mark.parametrize("seed", range(8))
def test_random_odd_shapes_fp32(seed):
    """Sizes as in the reference's GPU test (test_causal_product_gpu.py:47-54): E, M drawn
    from [10, 512), inputs U[0,1), L = 100; plus L values around the chunk size."""
    rng = np.random.RandomState(seed)
    E, M = int(rng.randint(10, 512)), int(rng.randint(10, 512))
    L = [100, 1, 31, 33, 130, 64, 257, 100][seed]
    N, H = (2, 3) if max(E, M) > 256 else (4, 10)
    g = torch.Generator().manual_seed(seed)
    Q, K, V, G = (torch.rand(N, H, L, d, generator=g) for d in (E, E, M, M))
    got = check_against_oracle(Q, K, V, G, "fp32")
    want = (orc.dense_forward(Q, K, V),) + tuple(orc.dense_backward(Q, K, V, G))
    for name, a, b in zip(("out", "gQ", "gK", "gV"), got, want):
        assert orc.max_relative_error(b, a) < 1e-5, name


def test_signed_inputs_and_many_segments_fp32():
    g = torch.Generator().manual_seed(11)
    Q, K, V, G = (torch.randn(1, 2, 3000, d, generator=g) for d in (48, 48, 80, 80))
    check_against_oracle(Q, K, V, G, "fp32", chunked=True)


def test_strided_views_fp32():
    """(N, L, H, dim) storage viewed as (N, H, L, dim), a sliced feature dimension and an
    expanded grad_out -- the reference only requires stride(3) == 1."""
    g = torch.Generator().manual_seed(12)
    N, H, L, D, M = 2, 3, 150, 32, 40
    Qs, Ks = (torch.rand(N, L, H, D + 8, generator=g) for _ in range(2))
    Vs = torch.rand(N, L, H, M, generator=g)
    Q, K, V = Qs.permute(0, 2, 1, 3)[..., 4:4 + D], Ks.permute(0, 2, 1, 3)[..., :D], Vs.permute(0, 2, 1, 3)
    Gd = torch.ones(1, 1, 1, 1).cuda().expand(N, H, L, M)
    Qd, Kd, Vd = (t.cuda().permute(0, 2, 1, 3) for t in (Qs, Ks, Vs))
    Qd, Kd = Qd[..., 4:4 + D], Kd[..., :D]
    assert not Qd.is_contiguous()
    Qd.requires_grad_(True), Kd.requires_grad_(True), Vd.requires_grad_(True)
    out = causal_dot_product(Qd, Kd, Vd)
    out.backward(Gd)
    want_o = orc.dense_forward(Q, K, V)
    want_g = orc.dense_backward(Q, K, V, torch.ones(N, H, L, M))
    assert orc.rel_err(out, want_o) < 1e-5
    for a, b in zip((Qd.grad, Kd.grad, Vd.grad), want_g):
        assert orc.rel_err(a, b) < 1e-5


def test_raw_native_signature_and_sum_backward():
    """The in-place native functions with the reference's argument lists."""
    g = torch.Generator().manual_seed(13)
    Q, K, V = (torch.rand(2, 2, 90, d, generator=g) for d in (16, 16, 24))
    Qd, Kd, Vd = dev(Q, K, V)
    out = torch.full((2, 2, 90, 24), float("nan"), device="cuda")
    causal_dot_product_cuda(Qd, Kd, Vd, out)
    assert orc.rel_err(out, orc.dense_forward(Q, K, V)) < 1e-5
    go = torch.rand(2, 2, 90, 24, generator=g)
    gq, gk, gv = (torch.full_like(t, float("nan")) for t in (Qd, Kd, Vd))
    causal_dot_backward_cuda(Qd, Kd, Vd, go.cuda(), gq, gk, gv)
    for a, b in zip((gq, gk, gv), orc.dense_backward(Q, K, V, go)):
        assert orc.rel_err(a, b) < 1e-5
    assert CausalDotProduct.dot["cuda"] is causal_dot_product_cuda


def test_empty_and_degenerate_shapes():
    for shape in [(0, 2, 5, 4, 4), (2, 0, 5, 4, 4), (2, 2, 0, 4, 4)]:
        N, H, L, D, M = shape
        Q = torch.rand(N, H, L, D, device="cuda", requires_grad=True)
        K = torch.rand(N, H, L, D, device="cuda", requires_grad=True)
        V = torch.rand(N, H, L, M, device="cuda", requires_grad=True)
        out = causal_dot_product(Q, K, V)
        assert out.shape == (N, H, L, M)
        out.sum().backward()
        assert Q.grad.shape == Q.shape
    # a single position attends to itself
    Q, K, V = (torch.rand(1, 1, 1, d) for d in (3, 3, 2))
    out = causal_dot_product(*dev(Q, K, V))
    assert orc.rel_err(out, orc.dense_forward(Q, K, V)) < 1e-6


def test_dtype_errors():
    x = torch.rand(1, 1, 4, 4, device="cuda")
    with pytest.raises(RuntimeError, match="Float"):
        causal_dot_product(x.double(), x.double(), x.double())
    with pytest.raises(RuntimeError, match="Float"):
        causal_dot_product(x.half(), x.half(), x.half())


def test_bf16_io_fp32_arithmetic():
    g = torch.Generator().manual_seed(14)
    Q, K, V, G = workloads.elu_inputs(1, 2, 700, 64, 64, g, torch.bfloat16)
    # inputs are exactly representable; only the bf16 rounding of the outputs remains
    check_against_oracle(Q, K, V, G, "fp32", chunked=True, tol=5e-3)


def test_states_split_sequence_fp32():
    """Two half-sequence calls chained through S / R states equal one full call."""
    g = torch.Generator().manual_seed(15)
    N, H, L, D, M = 1, 3, 1200, 32, 48
    Q, K, V, G = (torch.rand(N, H, L, d, generator=g) for d in (D, D, M, M))
    Qd, Kd, Vd, Gd = dev(Q, K, V, G)
    h = L // 2
    want_o = orc.chunked_forward(Q, K, V)
    want_g = orc.chunked_backward(Q, K, V, G)

    S0 = causal_state_sum(Kd[:, :, :h], Vd[:, :, :h])
    assert orc.rel_err(S0, orc.local_states(None, K[:, :, :h], V[:, :, :h])) < 1e-5
    o1 = torch.empty(N, H, h, M, device="cuda")
    fin = torch.empty(N, H, D, M, device="cuda")
    causal_dot_product_cuda(Qd[:, :, :h], Kd[:, :, :h], Vd[:, :, :h], o1, final_state=fin)
    assert orc.rel_err(fin, S0) < 1e-5
    o2 = torch.empty(N, H, L - h, M, device="cuda")
    fin2 = torch.empty(N, H, D, M, device="cuda")
    causal_dot_product_cuda(Qd[:, :, h:], Kd[:, :, h:], Vd[:, :, h:], o2, initial_state=fin,
                            final_state=fin2)
    assert orc.rel_err(torch.cat([o1, o2], 2), want_o) < 1e-5
    assert orc.rel_err(fin2, orc.local_states(None, K, V)) < 1e-5

    R1 = causal_state_sum(Qd[:, :, h:], Gd[:, :, h:])
    g1 = [torch.empty(N, H, h, d, device="cuda") for d in (D, D, M)]
    g2 = [torch.empty(N, H, L - h, d, device="cuda") for d in (D, D, M)]
    causal_dot_backward_cuda(Qd[:, :, :h], Kd[:, :, :h], Vd[:, :, :h], Gd[:, :, :h], *g1,
                             initial_grad_state=R1)
    causal_dot_backward_cuda(Qd[:, :, h:], Kd[:, :, h:], Vd[:, :, h:], Gd[:, :, h:], *g2,
                             initial_state=fin)
    for a, b, c in zip(g1, g2, want_g):
        assert orc.rel_err(torch.cat([a, b], 2), c) < 1e-5


def test_run_to_run_determinism():
    """No atomics anywhere: repeated runs must agree bit for bit."""
    Q, K, V, G = workloads.make_inputs(1)
    a = run_fwd_bwd(Q, K, V, G, "fp32")
    b = run_fwd_bwd(Q, K, V, G, "fp32")
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_workspace_error_code(native_lib):
    """Too small a workspace is refused with its own status and nothing is launched."""
    import ctypes
    from fast_transformers_b200 import _native
    Q = torch.rand(1, 1, 4096, 8, device="cuda")
    out = torch.zeros(1, 1, 4096, 8, device="cuda")
    s = _native.strides3(Q)
    st = native_lib.ftb_causal_dot_product(
        Q.data_ptr(), Q.data_ptr(), Q.data_ptr(), out.data_ptr(), 1, 1, 4096, 8, 8, s, s, s, s,
        _native.F32, _native.MODE_FP32_SIMT, None, None, 0, None, 0, None)
    assert st == _native.ERR_WORKSPACE
    torch.cuda.synchronize()
    assert out.abs().sum().item() == 0
    st = native_lib.ftb_causal_dot_product(
        Q.data_ptr(), Q.data_ptr(), Q.data_ptr(), out.data_ptr(), 1, 1, 16, 600, 8, s, s, s, s,
        _native.F32, _native.MODE_FP32_SIMT, None, None, 0, None, 0, None)
    assert st == _native.ERR_UNSUPPORTED


def test_linearity_property_config2_fp32():
    """Full-size config 2 (B8 H8 L4096 D=M=64): out is linear in V, and the last row of each
    head equals q_L . (K^T V), a size-independent check against one fp64 GEMM."""
    Q, K, V, G = workloads.make_inputs(2)
    Qd, Kd, Vd = dev(Q, K, V)
    o1 = causal_dot_product(Qd, Kd, Vd)
    o2 = causal_dot_product(Qd, Kd, 2.0 * Vd)
    assert orc.rel_err(o2, 2.0 * o1.double()) < 1e-6
    S = K.double().transpose(-1, -2) @ V.double()
    last = (Q[:, :, -1:].double() @ S)
    assert orc.rel_err(o1[:, :, -1:], last) < 1e-5
    first = (Q[:, :, :1].double() * K[:, :, :1].double()).sum(-1, keepdim=True) * V[:, :, :1].double()
    assert orc.rel_err(o1[:, :, :1], first) < 1e-6


@pytest.mark.parametrize("mode", ["fp32", "mma"])
def test_inputs_whose_last_dimension_is_not_contiguous(mode):
    """Q, K, V given as transposes (last stride != 1): the reference accepts any strides through
    its accessors (causal_product_cpu.cpp:88-99); here such inputs are copied row-major and the
    results come back in row-major buffers."""
    g = torch.Generator().manual_seed(77)
    N, H, L, D = 1, 2, 300, 64
    Qt, Kt, Vt, Gt = (torch.rand(N, H, D, L, generator=g) for _ in range(4))
    Q, K, V, G = (t.transpose(-1, -2) for t in (Qt, Kt, Vt, Gt))
    assert Q.stride(3) != 1
    q, k, v = (t.cuda().transpose(-1, -2).requires_grad_(True) for t in (Qt, Kt, Vt))
    with ftb.mode(mode):
        out = causal_dot_product(q, k, v)
        out.backward(Gt.cuda().transpose(-1, -2))
    torch.cuda.synchronize()
    want = (orc.dense_forward(Q, K, V),) + tuple(orc.dense_backward(Q, K, V, G))
    for name, a, b in zip(("out", "gQ", "gK", "gV"), (out, q.grad, k.grad, v.grad), want):
        assert orc.rel_err(a, b) < TOL[mode], name


@pytest.mark.parametrize("mode", ["fp32", "mma"])
def test_values_longer_than_queries_use_the_first_rows(mode):
    """The reference's layer passes all S rows of V when L < S and its kernels read the first L
    (tests/attention/test_causal_linear_attention.py:33-39); the gradient of the unread rows is 0."""
    g = torch.Generator().manual_seed(12)
    N, H, L, S, D = 1, 2, 200, 260, 64
    Q, K, G = (torch.rand(N, H, L, D, generator=g) for _ in range(3))
    V = torch.rand(N, H, S, D, generator=g)
    Qd, Kd, Vd, Gd = dev(Q, K, V, G)
    out = torch.empty(N, H, L, D, device="cuda")
    causal_dot_product_cuda(Qd, Kd, Vd, out, mode)
    gq, gk = torch.empty_like(Qd), torch.empty_like(Kd)
    gv = torch.full_like(Vd, float("nan"))
    causal_dot_backward_cuda(Qd, Kd, Vd, Gd, gq, gk, gv, mode)
    want = (orc.dense_forward(Q, K, V[:, :, :L]),) + tuple(orc.dense_backward(Q, K, V[:, :, :L], G))
    for name, a, b in zip(("out", "gQ", "gK", "gV"), (out, gq, gk, gv[:, :, :L]), want):
        assert orc.rel_err(a, b) < TOL[mode], name
    assert torch.all(gv[:, :, L:] == 0)


@pytest.mark.parametrize("mode", ["fp32", "mma"])
def test_concurrent_calls_from_two_threads_on_two_streams(mode):
    """The library is re-entrant: two host threads, each on a stream of its own, run forward and
    backward at the same time (as the caller's thread and the autograd thread do); the results are
    bitwise those of the same calls made one after the other."""
    import threading
    data = [dev(*workloads.make_inputs(1, trial=t)) for t in range(2)]

    def work(i, box):
        Q, K, V, G = data[i]
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(5):
                out = torch.empty_like(V)
                grads = [torch.empty_like(t) for t in (Q, K, V)]
                causal_dot_product_cuda(Q, K, V, out, mode)
                causal_dot_backward_cuda(Q, K, V, G, *grads, mode)
            stream.synchronize()
        box[i] = [out] + grads

    serial, parallel = [None, None], [None, None]
    for i in range(2):
        work(i, serial)
    threads = [threading.Thread(target=work, args=(i, parallel)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for a, b in zip(serial, parallel):
        for x, y in zip(a, b):
            assert torch.equal(x, y)


def test_ordinary_launches_give_the_same_results_as_programmatic_ones():
    """FTB200_NO_PDL=1 (ordinary launches instead of programmatic stream serialisation) in a child
    process: same kernels, same arithmetic, bitwise the same results -- for the 64-wide scans and
    for a wide feature dimension (three feature blocks)."""
    import os
    import subprocess
    import sys
    import tempfile
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import sys, torch; sys.path.insert(0, %r)\n"
        "import fast_transformers_b200 as ftb\n"
        "from fast_transformers_b200 import workloads\n"
        "from fast_transformers_b200.causal_product import causal_dot_product\n"
        "Q, K, V, G = (t.cuda() for t in workloads.make_inputs(1))\n"
        "Q.requires_grad_(True); K.requires_grad_(True); V.requires_grad_(True)\n"
        "with ftb.mode('mma'):\n"
        "    out = causal_dot_product(Q, K, V); out.backward(G)\n"
        "res = [out.detach().cpu(), Q.grad.cpu(), K.grad.cpu(), V.grad.cpu()]\n"
        "g = torch.Generator().manual_seed(3)\n"
        "Q, K = (torch.rand(1, 5, 2000, 192, generator=g).cuda().requires_grad_(True) for _ in range(2))\n"
        "V = torch.randn(1, 5, 2000, 64, generator=g).cuda().requires_grad_(True)\n"
        "with ftb.mode('mma'):\n"
        "    out = causal_dot_product(Q, K, V); out.backward(torch.ones_like(out))\n"
        "res += [out.detach().cpu(), Q.grad.cpu(), K.grad.cpu(), V.grad.cpu()]\n"
        "torch.cuda.synchronize(); ftb.check_device_status()\n"
        "torch.save(res, sys.argv[1])\n" % root)
    results = []
    with tempfile.TemporaryDirectory() as tmp:
        for flag in ("0", "1"):
            env = dict(os.environ)
            env.pop("FTB200_NO_PDL", None)
            if flag == "1":
                env["FTB200_NO_PDL"] = "1"
            path = os.path.join(tmp, "r%s.pt" % flag)
            subprocess.run([sys.executable, "-c", code, path], check=True, env=env, timeout=300)
            results.append(torch.load(path))
    for a, b in zip(*results):
        assert torch.equal(a, b)
