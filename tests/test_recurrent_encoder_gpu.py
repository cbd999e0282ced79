"""The recurrent encoder on the GPU: ``RecurrentEncoderBuilder`` models against the batch encoder
with the same weights (the method of the reference's tests/recurrent/test_transformer_encoder.py),
token by token from the start and after a prompt handed over by ``prefill``.  The file name sorts
after the kernel tests: it composes what they check one by one (batch layer, state sum, step)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import fast_transformers_b200 as ftb  # noqa: E402
from oracle import causal_oracle as orc  # noqa: E402
from fast_transformers_b200.builders import (RecurrentEncoderBuilder,  # noqa: E402
                                             TransformerEncoderBuilder)
from fast_transformers_b200.masking import LengthMask, TriangularCausalMask  # noqa: E402


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available()
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False      # the projections in full fp32 on both sides
    yield native_lib
    torch.backends.cuda.matmul.allow_tf32 = tf32
    torch.cuda.synchronize()
    assert native_lib.ftb_device_status(1) == 0


def _models(M):
    kw = dict(n_layers=2, n_heads=4, query_dimensions=16, value_dimensions=M,
              feed_forward_dimensions=64, attention_type="causal-linear", dropout=0.0)
    torch.manual_seed(11)
    batch = TransformerEncoderBuilder.from_kwargs(**kw).get().cuda().eval()
    rec = RecurrentEncoderBuilder.from_kwargs(**kw).get().cuda().eval()
    rec.load_state_dict(batch.state_dict())
    return batch, rec


@pytest.mark.parametrize("M", [16, 64])
@torch.no_grad()
def test_recurrent_encoder_equals_batch_encoder(M):
    batch, rec = _models(M)
    N, L = 3, 40
    x = torch.randn(N, L, 4 * M, device="cuda")
    with ftb.mode("fp32"):
        want = batch(x, attn_mask=TriangularCausalMask(L, device="cuda"))
    state, ys = None, []
    for i in range(L):
        y, state = rec(x[:, i], state)
        ys.append(y)
    assert orc.rel_err(torch.stack(ys, 1), want) < 1e-4


@torch.no_grad()
def test_prefill_then_decode_equals_batch_encoder():
    batch, rec = _models(16)
    N, L, P = 3, 40, 25
    x = torch.randn(N, L, 64, device="cuda")
    with ftb.mode("fp32"):
        want = batch(x, attn_mask=TriangularCausalMask(L, device="cuda"))
        y0, state = rec.prefill(x[:, :P])
    assert orc.rel_err(y0, want[:, :P]) < 1e-4
    ys = []
    for i in range(P, L):
        y, state = rec(x[:, i], state)
        ys.append(y)
    assert orc.rel_err(torch.stack(ys, 1), want[:, P:]) < 1e-4


@torch.no_grad()
def test_prefill_with_prompts_of_different_lengths():
    _, rec = _models(16)
    x = torch.randn(2, 12, 64, device="cuda")
    lengths = torch.tensor([12, 5], device="cuda")
    with ftb.mode("fp32"):
        _, state = rec.prefill(x, LengthMask(lengths, max_len=12))
        _, short = rec.prefill(x[1:, :5])
    for s_all, s_short in zip(state, short):
        assert orc.rel_err(s_all[0][1:], s_short[0]) < 1e-5
        assert orc.rel_err(s_all[1][1:], s_short[1]) < 1e-5


@torch.no_grad()
def test_against_the_reference_recurrent_encoder(golden):
    """The reference's RecurrentTransformerEncoder on the same weights and inputs
    (tests/golden/make_golden.py, ``recurrent_encoder``): outputs and per-layer states, token by
    token and with the first ``prefix`` positions handed over by ``prefill``."""
    g = golden("recurrent_encoder")
    T = lambda name: torch.from_numpy(np.asarray(g[name])).cuda()     # noqa: E731
    model = RecurrentEncoderBuilder.from_kwargs(
        n_layers=2, n_heads=4, query_dimensions=16, value_dimensions=16,
        feed_forward_dimensions=96, activation="gelu", dropout=0.0,
        attention_type="causal-linear").get().eval()
    model.load_state_dict({k[4:]: torch.from_numpy(np.asarray(g[k])) for k in g.files
                           if k.startswith("sd__")})
    model = model.cuda()
    x, want, P = T("x"), T("y"), int(g["prefix"])
    state, ys = None, []
    for i in range(x.shape[1]):
        y, state = model(x[:, i], state)
        ys.append(y)
    assert orc.rel_err(torch.stack(ys, 1), want) < 1e-4
    for layer, (S, z) in enumerate(state):
        assert orc.rel_err(S, T("end_S%d" % layer)) < 1e-4
        assert orc.rel_err(z, T("end_z%d" % layer)) < 1e-4
    with ftb.mode("fp32"):
        y0, state = model.prefill(x[:, :P])
    assert orc.rel_err(y0, want[:, :P]) < 1e-4
    for layer, (S, z) in enumerate(state):
        assert orc.rel_err(S, T("mid_S%d" % layer)) < 1e-4
        assert orc.rel_err(z, T("mid_z%d" % layer)) < 1e-4
