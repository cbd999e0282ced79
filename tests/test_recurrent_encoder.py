"""Host logic of the recurrent encoder (projection layer, encoder layer, encoder, builder,
prefill) on the CPU.  The native kernels need a GPU, so here the four native calls the modules
make are replaced by the oracle's restatements of them (same argument and result layouts); what
is under test is everything around them: head splitting, residuals and norms, which state goes to
which layer, the hand-over from ``prefill`` to the steps, and the interchange of weights with the
batch encoder.  Method of the reference's tests/recurrent/test_transformer_encoder.py (batch
model against the recurrent model on the same weights)."""
import numpy as np
import pytest
import torch

import fast_transformers_b200  # noqa: F401
from fast_transformers_b200.attention import causal_linear_attention as batch_mod
from fast_transformers_b200.builders import RecurrentEncoderBuilder, TransformerEncoderBuilder
from fast_transformers_b200.masking import LengthMask, TriangularCausalMask
from fast_transformers_b200.recurrent.attention.self_attention import linear_attention as rec_mod
from fast_transformers_b200.recurrent.transformers import RecurrentTransformerEncoder
import fast_transformers_b200.causal_product as cp_mod
from oracle import causal_oracle as orc


def _product(Q, K, V):
    return orc.chunked_forward(Q, K, V).to(Q.dtype)


def _normaliser(Q, K):
    return orc.normaliser(Q, K).to(Q.dtype)


def _state_sum(x, y, mode=None, workspace=None, reverse=False):
    return torch.einsum("nhld,nhlm->nhdm", x.double(), y.double()).float().contiguous()


def _step(Q, K, value, S, z, eps=1e-6, elu_plus_one=False):
    feature = orc.elu_features if elu_plus_one else (lambda t: t)
    y, (S2, z2) = orc.recurrent_step(Q, K, value, [S, z], feature=feature, eps=eps)
    S.copy_(S2)           # the native step updates the state in place
    z.copy_(z2)
    return y.to(Q.dtype)


@pytest.fixture()
def oracle_kernels(monkeypatch):
    monkeypatch.setattr(batch_mod, "causal_dot_product", _product)
    monkeypatch.setattr(batch_mod, "causal_normaliser", _normaliser)
    monkeypatch.setattr(cp_mod, "causal_state_sum", _state_sum)
    monkeypatch.setattr(rec_mod, "recurrent_linear_step", _step)


def _models(M=8, **extra):
    kw = dict(n_layers=3, n_heads=2, query_dimensions=8, value_dimensions=M,
              feed_forward_dimensions=32, attention_type="causal-linear", dropout=0.0)
    kw.update(extra)
    torch.manual_seed(0)
    batch = TransformerEncoderBuilder.from_kwargs(**kw).get().eval()
    rec = RecurrentEncoderBuilder.from_kwargs(**kw).get().eval()
    rec.load_state_dict(batch.state_dict())
    return batch, rec


def test_builder_and_state_dict_interchange():
    batch, rec = _models()
    assert isinstance(rec, RecurrentTransformerEncoder) and len(rec.layers) == 3
    assert list(rec.state_dict().keys()) == list(batch.state_dict().keys())
    with pytest.raises(ValueError):
        RecurrentEncoderBuilder.from_kwargs(attention_type="full")        # not in this registry
    b = RecurrentEncoderBuilder.from_kwargs(attention_type="linear", query_dimensions=8,
                                            final_normalization=False)
    assert b.get().norm is None


@pytest.mark.parametrize("M", [8, 64])     # 8: ones-column normaliser; 64: the separate one
@torch.no_grad()
def test_recurrent_encoder_equals_batch_encoder(oracle_kernels, M):
    batch, rec = _models(M=M)
    N, L = 2, 9
    x = torch.randn(N, L, 2 * M)
    want = batch(x, attn_mask=TriangularCausalMask(L))
    state, ys = None, []
    for i in range(L):
        y, state = rec(x[:, i], state)
        ys.append(y)
    assert len(state) == 3 and all(len(s) == 2 for s in state)
    assert orc.rel_err(torch.stack(ys, 1), want) < 1e-5


@torch.no_grad()
def test_prefill_then_decode_equals_batch_encoder(oracle_kernels):
    batch, rec = _models()
    N, L, P = 2, 11, 7
    x = torch.randn(N, L, 16)
    want = batch(x, attn_mask=TriangularCausalMask(L))
    y0, state = rec.prefill(x[:, :P])
    assert orc.rel_err(y0, want[:, :P]) < 1e-5
    ys = []
    for i in range(P, L):
        y, state = rec(x[:, i], state)
        ys.append(y)
    assert orc.rel_err(torch.stack(ys, 1), want[:, P:]) < 1e-5


@torch.no_grad()
def test_prefill_with_prompts_of_different_lengths(oracle_kernels):
    """Sequence 1's prompt is 4 positions, padded to 7: its state must stop at position 3, so
    decoding it from there equals decoding after an unpadded 4-position prompt."""
    _, rec = _models()
    x = torch.randn(2, 7, 16)
    lengths = torch.tensor([7, 4])
    _, state = rec.prefill(x, LengthMask(lengths, max_len=7))
    _, short = rec.prefill(x[1:, :4])
    for s_all, s_short in zip(state, short):
        assert orc.rel_err(s_all[0][1:], s_short[0]) < 1e-6
        assert orc.rel_err(s_all[1][1:], s_short[1]) < 1e-6


def test_memory_is_the_old_name_of_state(oracle_kernels):
    _, rec = _models()
    x = torch.randn(2, 16)
    with torch.no_grad():
        _, state = rec(x)
        with pytest.warns(DeprecationWarning):
            y1, _ = rec(x, memory=[[t.clone() for t in s] for s in state])
        y2, _ = rec(x, state)
    assert torch.equal(y1, y2)


def _golden_model(g):
    model = RecurrentEncoderBuilder.from_kwargs(
        n_layers=2, n_heads=4, query_dimensions=16, value_dimensions=16,
        feed_forward_dimensions=96, activation="gelu", dropout=0.0,
        attention_type="causal-linear").get().eval()
    model.load_state_dict({k[4:]: torch.from_numpy(np.asarray(g[k])) for k in g.files
                           if k.startswith("sd__")})
    return model


@torch.no_grad()
def test_against_the_reference_recurrent_encoder(oracle_kernels, golden):
    """Weights, inputs, outputs and states of the reference's RecurrentTransformerEncoder
    (tests/golden/make_golden.py, ``recurrent_encoder``): token by token, and with the first
    ``prefix`` positions handed over by ``prefill``."""
    g = golden("recurrent_encoder")
    T = lambda name: torch.from_numpy(np.asarray(g[name]))     # noqa: E731
    model, x, want, P = _golden_model(g), T("x"), T("y"), int(g["prefix"])
    state, ys = None, []
    for i in range(x.shape[1]):
        y, state = model(x[:, i], state)
        ys.append(y)
    assert orc.rel_err(torch.stack(ys, 1), want) < 1e-5
    for layer, (S, z) in enumerate(state):
        assert orc.rel_err(S, T("end_S%d" % layer)) < 1e-5
        assert orc.rel_err(z, T("end_z%d" % layer)) < 1e-5

    y0, state = model.prefill(x[:, :P])
    assert orc.rel_err(y0, want[:, :P]) < 1e-5
    for layer, (S, z) in enumerate(state):
        assert orc.rel_err(S, T("mid_S%d" % layer)) < 1e-5
        assert orc.rel_err(z, T("mid_z%d" % layer)) < 1e-5
    ys = []
    for i in range(P, x.shape[1]):
        y, state = model(x[:, i], state)
        ys.append(y)
    assert orc.rel_err(torch.stack(ys, 1), want[:, P:]) < 1e-5
