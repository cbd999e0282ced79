"""Host-side logic that needs no GPU: ABI surface, registry/builder behaviour, masks,
feature maps, error behaviour of the operator on CPU tensors."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import fast_transformers_b200 as ftb
from fast_transformers_b200 import _native
from fast_transformers_b200.attention import AttentionLayer, CausalLinearAttention
from fast_transformers_b200.attention_registry import AttentionRegistry, Int, Optional, Callable
from fast_transformers_b200.builders import AttentionBuilder, TransformerEncoderBuilder
from fast_transformers_b200.causal_product import CausalDotProduct, causal_dot_product
from fast_transformers_b200.events import EventDispatcher, QKVEvent, IntermediateOutput
from fast_transformers_b200.feature_maps import Favor, elu_feature_map
from fast_transformers_b200.masking import FullMask, LengthMask, TriangularCausalMask

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(native_lib):
    header = open(os.path.join(ROOT, "include", "ftb200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(ftb_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_native.EXPORTS)
    for name in declared:
        assert getattr(native_lib, name) is not None
    assert native_lib.ftb_version() >= 1000
    assert native_lib.ftb_status_string(0) == b"ok"
    assert b"workspace" in native_lib.ftb_status_string(_native.ERR_WORKSPACE)


def test_workspace_query_is_a_pure_function(native_lib):
    a = native_lib.ftb_causal_workspace_bytes(8, 8, 4096, 64, 64, 0, 0, 1, 0)
    b = native_lib.ftb_causal_workspace_bytes(8, 8, 4096, 64, 64, 0, 0, 1, 0)
    assert a == b and a > 0 and a % 256 == 0
    assert native_lib.ftb_causal_workspace_bytes(0, 8, 4096, 64, 64, 0, 0, 0, 0) == 0
    ws = native_lib.ftb_causal_workspace_bytes
    # tensor-core mode, wide fp32 shapes: whole [D][M] state blocks, forward one set, backward two
    fwd, bwd = ws(4, 12, 16384, 256, 64, 0, _native.MODE_MMA, 0, 0), ws(4, 12, 16384, 256, 64, 0, _native.MODE_MMA, 1, 0)
    assert fwd > 0 and fwd % (256 * 64 * 4) == 0 and bwd == 2 * fwd
    assert ws(2, 2, 4096, 128, 128, 0, _native.MODE_MMA, 1, 0) % (128 * 128 * 4) == 0
    # the split-operand mode: fp32 D = M = 64 only (0: nothing to allocate for a shape it refuses)
    x3 = ws(8, 8, 4096, 64, 64, 0, _native.MODE_MMA_X3, 1, 0)
    assert x3 > 0 and x3 % (2 * 64 * 64 * 4) == 0
    assert ws(8, 8, 4096, 32, 32, 0, _native.MODE_MMA_X3, 1, 0) == 0
    assert ws(8, 8, 4096, 64, 64, 1, _native.MODE_MMA_X3, 1, 0) == 0


def test_cpu_tensors_are_rejected_loudly():
    Q = torch.rand(1, 1, 4, 3)
    with pytest.raises(RuntimeError, match="CUDA"):
        causal_dot_product(Q, Q, Q)
    assert set(CausalDotProduct.dot) == {"cpu", "cuda"}
    assert set(CausalDotProduct.dot_backward) == {"cpu", "cuda"}


def test_mode_setting():
    assert ftb.get_mode() in ("fp32", "mma", "tf32x3")
    before = ftb.get_mode()
    with ftb.mode("mma"):
        assert ftb.get_mode() == "mma"
    assert ftb.get_mode() == before
    with ftb.mode("tf32x3"):
        assert ftb.get_mode() == "tf32x3"
        # the tier's name resolves to the split-operand kernels only where the caller says they apply
        from fast_transformers_b200.causal_product import _mode_id
        assert _mode_id(None, True) == _native.MODE_MMA_X3 and _mode_id(None) == _native.MODE_FP32_SIMT
    with pytest.raises(ValueError):
        ftb.set_mode("fp16")


def test_registry_entry_and_specs():
    cls, params = AttentionRegistry["causal-linear"]
    assert cls is CausalLinearAttention
    assert params == ["query_dimensions", "feature_map", "event_dispatcher"]
    with pytest.raises(ValueError):
        AttentionRegistry.register("causal-linear", CausalLinearAttention, [])
    with pytest.raises(ValueError):
        AttentionRegistry.validate_parameter("query_dimensions", "x")
    assert AttentionRegistry.validate_parameter("feature_map", None) is None
    assert Optional(Int, 3).get(None) == 3
    with pytest.raises(ValueError):
        Callable.get(3)


def test_attention_builder():
    b = AttentionBuilder.from_kwargs(query_dimensions=16)
    att = b.get("causal-linear")
    assert isinstance(att, CausalLinearAttention)
    with pytest.raises(ValueError):
        b.get("no-such-attention")
    with pytest.raises(ValueError):
        AttentionBuilder.from_kwargs(not_a_parameter=1)
    AttentionBuilder.from_kwargs(not_a_parameter=1, strict=False)
    b.feature_map = Favor.factory(n_dims=32)
    assert isinstance(b.get("causal-linear").feature_map, Favor)


def test_encoder_builder_defaults_and_strictness():
    b = TransformerEncoderBuilder()
    assert (b.n_layers, b.n_heads, b.query_dimensions, b.value_dimensions,
            b.feed_forward_dimensions, b.dropout, b.activation, b.final_normalization) == \
        (4, 4, 64, 64, 1024, 0.1, "relu", True)
    assert b.model_dimensions == 256
    with pytest.raises(ValueError):
        b.attention_type = "nope"
    with pytest.raises(ValueError):
        b.activation = "tanh"
    with pytest.raises(ValueError):
        TransformerEncoderBuilder.from_kwargs(foo=3)
    import argparse
    ns = argparse.Namespace(n_layers=2, unrelated=5, attention_type="causal-linear")
    b2 = TransformerEncoderBuilder.from_namespace(ns)
    assert b2.n_layers == 2 and b2.attention_type == "causal-linear"
    b3 = TransformerEncoderBuilder.from_kwargs(
        n_layers=3, n_heads=2, query_dimensions=8, value_dimensions=8,
        feed_forward_dimensions=16, attention_type="causal-linear", dropout=0.0)
    model = b3.get()
    assert len(model.layers) == 3
    assert isinstance(model.layers[0].attention, AttentionLayer)
    assert isinstance(model.layers[0].attention.inner_attention, CausalLinearAttention)
    assert model.layers[0].attention.query_projection.out_features == 16
    assert model.norm is not None


def test_encoder_state_dict_keys_match_reference(golden):
    g = golden("encoder")
    ref_keys = sorted(k[4:] for k in g.files if k.startswith("sd__"))
    model = TransformerEncoderBuilder.from_kwargs(
        n_layers=2, n_heads=4, query_dimensions=8, value_dimensions=8,
        feed_forward_dimensions=64, attention_type="causal-linear", dropout=0.0).get()
    assert sorted(model.state_dict().keys()) == ref_keys


def test_masks():
    m = TriangularCausalMask(5)
    assert m.lower_triangular and m.shape == (5, 5)
    assert torch.equal(m.bool_matrix, torch.tril(torch.ones(5, 5)).bool())
    assert not FullMask(4).lower_triangular
    assert FullMask(torch.tril(torch.ones(4, 4)).bool()).lower_triangular
    lm = LengthMask(torch.tensor([3, 1]), max_len=4)
    assert lm.float_matrix.tolist() == [[1, 1, 1, 0], [1, 0, 0, 0]]
    with pytest.raises(ValueError):
        FullMask(torch.ones(2, 2))
    bad = FullMask(torch.tensor([[True, False, True]]))
    with pytest.raises(ValueError):
        bad.lengths


def test_causal_layer_rejects_non_causal_mask():
    att = CausalLinearAttention(4)
    x = torch.rand(1, 3, 2, 4)
    lm = LengthMask(torch.tensor([3]))
    with pytest.raises(RuntimeError, match="lower triangular"):
        att(x, x, x, FullMask(3), lm, lm)


def test_feature_maps_cpu(golden):
    g = golden("favor")
    x, omega = torch.from_numpy(g["x"]), torch.from_numpy(g["omega"])
    f = Favor(16, n_dims=64)
    f.omega.copy_(omega)
    np.testing.assert_allclose(f(x).numpy(), g["phi"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(elu_feature_map(16)(x).numpy(), g["elu"], rtol=1e-6)
    f2 = Favor(16, n_dims=64, deterministic_eval=True).eval()
    f2.new_feature_map("cpu")
    assert torch.count_nonzero(f2.omega) == 0
    f2.train()
    f2.new_feature_map("cpu")
    assert torch.count_nonzero(f2.omega) > 0
    # columns inside one block are orthogonal
    w = f2.omega[:, :16]
    gram = w.t() @ w
    off = gram - torch.diag(torch.diag(gram))
    assert off.abs().max() < 1e-3 * gram.abs().max()


def test_events():
    ed = EventDispatcher()
    seen = []
    ed.listen(QKVEvent, lambda ev: seen.append(ev))
    ed.dispatch(IntermediateOutput(None, 1))
    ed.dispatch(QKVEvent(None, 1, 2, 3))
    assert len(seen) == 1 and seen[0].values == 3
    assert EventDispatcher.get("") is EventDispatcher.get("")
    assert EventDispatcher.get(ed) is ed


def test_recurrent_registry_entry_and_host_checks():
    """The recurrent mirror: registry key "linear" with the reference's parameter list
    (recurrent/attention/self_attention/linear_attention.py:95-102), the deprecated ``memory``
    argument, and the loud refusals (CPU tensors, gradients)."""
    import warnings
    from fast_transformers_b200.attention_registry import RecurrentAttentionRegistry
    from fast_transformers_b200.recurrent.attention import RecurrentLinearAttention
    from fast_transformers_b200.recurrent._utils import check_state
    assert "linear" in RecurrentAttentionRegistry.keys
    cls, params = RecurrentAttentionRegistry["linear"]
    assert cls is RecurrentLinearAttention
    assert RecurrentAttentionRegistry["causal-linear"][0] is RecurrentLinearAttention
    assert params == ["query_dimensions", "feature_map", "event_dispatcher"]
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        assert check_state(None, [1, 2]) == [1, 2]
        assert any(issubclass(x.category, DeprecationWarning) for x in w)
    att = RecurrentLinearAttention(8)
    q, k, v = torch.rand(2, 3, 8), torch.rand(2, 3, 8), torch.rand(2, 3, 5)
    with pytest.raises(RuntimeError):
        att(q.requires_grad_(True), k, v)          # no gradients through the native step
    with torch.no_grad(), pytest.raises(RuntimeError):
        att(q, k, v)                               # CPU tensors: there is no CPU path


def test_kernel_kind_table_matches_header():
    """The names ftb_timing_read's slots are reported under follow the header's FTB_KERNEL_*."""
    header = open(os.path.join(ROOT, "include", "ftb200.h")).read()
    kinds = dict(re.findall(r"#define FTB_KERNEL_([A-Z_0-9]+)\s+(\d+)", header))
    count = int(kinds.pop("KINDS"))
    assert count == len(_native.KERNEL_KINDS)
    for name, idx in kinds.items():
        assert _native.KERNEL_KINDS[int(idx)] == name.lower()


def test_exchange_buffer_size_and_argument_checks():
    """ftb_exchange_bytes is a pure function of (ranks, state elements): a 512-byte control block,
    2 x ranks counters rounded up to 256 bytes, 2 x ranks slots; 0 for what the exchange refuses."""
    lib = _native.lib()
    assert lib.ftb_exchange_bytes(8, 262144) == 512 + 256 + 2 * 8 * 262144 * 4
    assert lib.ftb_exchange_bytes(16, 4) == 512 + 256 + 2 * 16 * 4 * 4
    assert lib.ftb_exchange_bytes(17, 4) == 0          # more than 16 ranks
    assert lib.ftb_exchange_bytes(2, 6) == 0           # states move 16 bytes at a time
    assert lib.ftb_exchange_push(None, 4, None, 0, 2, 0, None) == _native.ERR_INVALID
    assert lib.ftb_exchange_receive(None, None, 4, 0, 2, 0, None) == _native.ERR_INVALID


def test_exchange_protocol_two_slots_suffice():
    """A model of the peer-memory exchange (csrc/rank_exchange.cuh): every rank runs
    push(e), receive(e), push(e+1), ... in order; a push writes slot[e & 1][src] and then
    flag[e & 1][src] = e in the buffers of the ranks it feeds, once each of them has finished
    its receive of e - 2; a receive can run once the flags of its sources have reached e.  Ranks
    advance in random order as far as those rules allow, with any sequence of directions
    (alternating as in training, or forward only).  Whatever the interleaving, a receive must
    find the values of ITS exchange in the slots, and everybody must get to the end."""
    import random
    rng = random.Random(5)
    for world in (2, 3, 5):
        for trial in range(150):
            exchanges = 7
            directions = [rng.random() < (0.5 if trial % 3 else 0.0) for _ in range(exchanges)]
            slot = [[[None] * world for _ in range(2)] for _ in range(world)]   # [owner][parity][src]
            flag = [[[0] * world for _ in range(2)] for _ in range(world)]
            received = [0] * world
            pc = [0] * world            # operations completed per rank: push, receive, push, ...
            idle = 0
            while any(c < exchanges * 2 for c in pc):
                r = rng.randrange(world)
                idle += 1
                assert idle < 100000, "stuck"
                if pc[r] >= exchanges * 2:
                    continue
                e, reverse = pc[r] // 2 + 1, directions[pc[r] // 2]
                feeds = range(0, r) if reverse else range(r + 1, world)
                sources = range(r + 1, world) if reverse else range(0, r)
                if pc[r] % 2 == 0:                                      # push(e)
                    if any(received[p] + 2 < e for p in feeds):
                        continue                                        # a slot is still in use
                    for p in feeds:
                        slot[p][e & 1][r] = (r, e)
                        flag[p][e & 1][r] = e
                else:                                                   # receive(e)
                    if any(flag[r][e & 1][p] < e for p in sources):
                        continue                                        # still waiting
                    assert all(slot[r][e & 1][p] == (p, e) for p in sources), (world, trial, r, e)
                    received[r] = e
                pc[r] += 1
                idle = 0
