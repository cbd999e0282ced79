"""The recurrent step (``ftb_recurrent_linear_step`` behind ``RecurrentLinearAttention``) against
the reference module's outputs (golden fixture), the fp64 oracle, and the batch form."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import causal_oracle as orc  # noqa: E402
from fast_transformers_b200.attention import CausalLinearAttention  # noqa: E402
from fast_transformers_b200.feature_maps import Favor  # noqa: E402
from fast_transformers_b200.masking import LengthMask, TriangularCausalMask  # noqa: E402
from fast_transformers_b200.recurrent.attention import RecurrentLinearAttention  # noqa: E402
from fast_transformers_b200.recurrent.attention.self_attention.linear_attention import (  # noqa: E402
    recurrent_linear_step)


def T(a):
    return torch.from_numpy(np.asarray(a))


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available()
    yield native_lib
    torch.cuda.synchronize()
    assert native_lib.ftb_device_status(1) == 0


@torch.no_grad()
def test_steps_match_reference_module(golden):
    g = golden("recurrent")
    q, k, v = (T(g[n]).cuda() for n in "qkv")
    L = q.shape[1]
    att = RecurrentLinearAttention(q.shape[3])
    for tag, state in (("empty", None), ("given", [T(g["S0"]).cuda(), T(g["z0"]).cuda()])):
        ys = []
        for i in range(L):
            y, state = att(q[:, i], k[:, i], v[:, i], state)
            assert y.shape == (q.shape[0], q.shape[2], v.shape[3]) and len(state) == 2
            ys.append(y)
        # the reference's own bound for this module (test_linear_attention.py:79)
        assert (torch.stack(ys, 1).cpu() - T(g[tag + "_y"])).abs().max() < 1e-5
        assert orc.rel_err(state[0], T(g[tag + "_S"])) < 1e-5
        assert orc.rel_err(state[1], T(g[tag + "_z"])) < 1e-5


@torch.no_grad()
def test_batch_form_equals_recurrent_form():
    """The reference's test_correctness (test_linear_attention.py:54-79) on the GPU: the batch
    layer (tcgen05 or CUDA-core product) against 100 native steps, bound 1e-5."""
    torch.manual_seed(4)
    N, H, E, M, L = 10, 4, 25, 64, 100
    q, k, v = (torch.rand(N, L, H, d, device="cuda") for d in (E, E, M))
    lm = LengthMask(torch.full((N,), L, dtype=torch.long, device="cuda"))
    v1 = CausalLinearAttention(E).eval()(q, k, v, TriangularCausalMask(L, device="cuda"), lm, lm)
    rec = RecurrentLinearAttention(E).eval()
    state, ys = None, []
    for i in range(L):
        y, state = rec(q[:, i], k[:, i], v[:, i], state)
        ys.append(y)
    assert (v1 - torch.stack(ys, 1)).abs().max() < 1e-5


@torch.no_grad()
@pytest.mark.parametrize("N,H,E,M", [(1, 1, 1, 1), (3, 2, 19, 33), (2, 3, 64, 300), (1, 2, 512, 64)])
def test_step_against_fp64_oracle_odd_shapes(N, H, E, M):
    g = torch.Generator().manual_seed(E * 1000 + M)
    q, k = (torch.randn(N, H, E, generator=g) for _ in range(2))
    v = torch.randn(N, H, M, generator=g)
    S, z = torch.rand(N, H, E, M, generator=g), torch.rand(N, H, E, generator=g) + 0.5
    want_y, (want_S, want_z) = orc.recurrent_step(q, k, v, [S, z])
    # strided inputs: slices of a larger (N, L, H, dim) buffer, as a decoder passes them
    big = torch.zeros(N, 3, H, E).cuda()
    big[:, 1] = q.cuda()
    Sd, zd = S.cuda(), z.cuda()
    att = RecurrentLinearAttention(E)
    y, state = att(big[:, 1], k.cuda(), v.cuda(), [Sd, zd])
    assert state[0] is Sd and state[1] is zd          # updated in place
    assert orc.rel_err(y, want_y) < 1e-5
    assert orc.rel_err(Sd, want_S) < 1e-5 and orc.rel_err(zd, want_z) < 1e-5
    # features given directly (no map inside the kernel) give the same numbers
    Sd2, zd2 = S.cuda(), z.cuda()
    y2 = recurrent_linear_step(orc.elu_features(q).float().cuda(), orc.elu_features(k).float().cuda(),
                               v.cuda(), Sd2, zd2, 1e-6, elu_plus_one=False)
    assert orc.rel_err(y2, want_y) < 1e-5 and orc.rel_err(Sd2, want_S) < 1e-5


@torch.no_grad()
def test_prefill_in_batch_form_then_decode():
    """Prefix through the batch layer, state handed over, the rest token by token: equal to the
    batch layer over the whole sequence.  Also with a non-default feature map (Favor)."""
    torch.manual_seed(7)
    N, H, E, M, L, P = 2, 3, 16, 24, 40, 29
    for fmap in (None, Favor.factory(n_dims=32, redraw=10 ** 9)):
        q, k, v = (torch.randn(N, L, H, d, device="cuda") * 0.5 for d in (E, E, M))
        batch = CausalLinearAttention(E, feature_map=fmap).cuda().eval()
        rec = RecurrentLinearAttention(E, feature_map=fmap).cuda().eval()
        if fmap is not None:
            batch.feature_map.new_feature_map("cuda")
            rec.feature_map.omega.copy_(batch.feature_map.omega)
        lm = LengthMask(torch.full((N,), L, dtype=torch.long, device="cuda"))
        full = batch(q, k, v, TriangularCausalMask(L, device="cuda"), lm, lm)
        if fmap is not None:
            # new_feature_map redraws omega inside state_after / forward(state=None): keep ours
            omega = batch.feature_map.omega.clone()
            rec.feature_map.new_feature_map = lambda device: None
            rec.feature_map.omega.copy_(omega)
        state = rec.state_after(k[:, :P], v[:, :P])
        ys = []
        for i in range(P, L):
            y, state = rec(q[:, i], k[:, i], v[:, i], state)
            ys.append(y)
        assert orc.rel_err(torch.stack(ys, 1), full[:, P:]) < 2e-5


def test_status_codes(native_lib):
    from fast_transformers_b200 import _native
    q = torch.rand(1, 1, 600, device="cuda")
    v = torch.rand(1, 1, 8, device="cuda")
    S, z = torch.zeros(1, 1, 600, 8, device="cuda"), torch.zeros(1, 1, 600, device="cuda")
    with pytest.raises(_native.NativeError) as e:
        recurrent_linear_step(q, q, v, S, z)
    assert e.value.status == _native.ERR_UNSUPPORTED      # D > 512
    with pytest.raises(RuntimeError):
        recurrent_linear_step(q.double(), q.double(), v.double(), S, z)
    empty = recurrent_linear_step(torch.rand(0, 2, 4, device="cuda"), torch.rand(0, 2, 4, device="cuda"),
                                  torch.rand(0, 2, 3, device="cuda"), torch.zeros(0, 2, 4, 3, device="cuda"),
                                  torch.zeros(0, 2, 4, device="cuda"))
    assert empty.shape == (0, 2, 3)
