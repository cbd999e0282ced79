"""The oracle against the reference's outputs (golden fixtures) and against itself."""
import numpy as np
import pytest
import torch

from oracle import causal_oracle as orc
from fast_transformers_b200 import workloads


def T(a):
    return torch.from_numpy(np.asarray(a))


def test_c_port_is_bit_exact_with_reference_small(golden):
    g = golden("product_small")
    Q, K, V, G = (T(g[k]) for k in "QKVG")
    out = orc.c_forward(Q, K, V, "f32")
    gQ, gK, gV = orc.c_backward(Q, K, V, G, "f32")
    # same recurrence, same summation order, same fp32 arithmetic: the sequential port must
    # reproduce the reference extension bit for bit
    assert torch.equal(out, T(g["out"]))
    assert torch.equal(gQ, T(g["gQ"])) and torch.equal(gK, T(g["gK"])) and torch.equal(gV, T(g["gV"]))


def test_fp64_forms_agree_and_match_reference_small(golden):
    g = golden("product_small")
    Q, K, V, G = (T(g[k]) for k in "QKVG")
    dense = orc.dense_forward(Q, K, V)
    assert orc.rel_err(orc.chunked_forward(Q, K, V, chunk=16), dense) < 1e-13
    assert orc.rel_err(orc.c_forward(Q, K, V, "f64"), dense) < 1e-13
    assert orc.rel_err(T(g["out"]), dense) < 1e-6
    # the reference tests' own criterion (test_causal_product_cpu.py:49)
    assert orc.max_relative_error(dense, T(g["out"])) < 1e-5
    dg = orc.dense_backward(Q, K, V, G)
    cg = orc.chunked_backward(Q, K, V, G, chunk=16)
    c64 = orc.c_backward(Q, K, V, G, "f64")
    for name, d, c, c6 in zip(("gQ", "gK", "gV"), dg, cg, c64):
        assert orc.rel_err(c, d) < 1e-13
        assert orc.rel_err(c6, d) < 1e-13
        assert orc.rel_err(T(g[name]), d) < 1e-6
        assert orc.max_relative_error(d, T(g[name])) < 1e-5


def test_config1_oracle_vs_reference_sample(golden):
    g = golden("product_config1_sample")
    Q, K, V, G = workloads.make_inputs(1)
    rows = T(g["rows"])
    out = orc.chunked_forward(Q, K, V)
    gQ, gK, gV = orc.chunked_backward(Q, K, V, G)
    for name, x in (("out", out), ("gQ", gQ), ("gK", gK), ("gV", gV)):
        ref = T(g[name])
        assert orc.rel_err(ref, x[:, :, rows]) < 2e-6, name
    sums = [t.sum().item() for t in (out, gQ, gK, gV)]
    np.testing.assert_allclose(sums, g["checksum"], rtol=1e-5)


def test_config1_c_port_vs_reference_sample(golden):
    g = golden("product_config1_sample")
    Q, K, V, G = workloads.make_inputs(1)
    rows = T(g["rows"])
    out = orc.c_forward(Q, K, V)
    gQ, gK, gV = orc.c_backward(Q, K, V, G)
    for name, x in (("out", out), ("gQ", gQ), ("gK", gK), ("gV", gV)):
        assert torch.equal(x[:, :, rows], T(g[name])), name


def test_reference_extension_matches_golden_when_built(golden):
    if orc.reference_ext() is None:
        pytest.skip("oracle/_ref not built (no reference checkout)")
    g = golden("product_small")
    Q, K, V, G = (T(g[k]) for k in "QKVG")
    assert torch.equal(orc.reference_forward(Q, K, V), T(g["out"]))
    gq, gk, gv = orc.reference_backward(Q, K, V, G)
    assert torch.equal(gq, T(g["gQ"])) and torch.equal(gk, T(g["gK"])) and torch.equal(gv, T(g["gV"]))


@pytest.mark.parametrize("case", ["eq", "lt", "gt"])
def test_layer_oracle_vs_reference(golden, case):
    g = golden("layer")
    q, k, v = (T(g[case + "_" + n]) for n in "qkv")
    y = orc.layer_forward(q, k, v, key_lengths=T(g[case + "_klen"]))
    assert orc.rel_err(T(g[case + "_y"]), y) < 1e-5


def test_feature_maps_vs_reference(golden):
    g = golden("favor")
    x, omega = T(g["x"]), T(g["omega"])
    assert orc.rel_err(T(g["phi"]), orc.favor_features(x.double(), omega.double())) < 1e-6
    assert orc.rel_err(T(g["elu"]), orc.elu_features(x.double())) < 1e-6
    # the package's own CPU-side generator used for config 5 inputs
    assert orc.rel_err(workloads.favor_map(x, omega), T(g["phi"])) < 1e-6


def test_states_compose():
    """S_init / R_init make two half-range calls equal one full-range call."""
    g = torch.Generator().manual_seed(5)
    Q, K, V, G = (torch.rand(1, 2, 48, d, generator=g) for d in (5, 5, 7, 7))
    full = orc.chunked_forward(Q, K, V, chunk=8)
    S0 = orc.local_states(None, K[:, :, :24], V[:, :, :24])
    second = orc.chunked_forward(Q[:, :, 24:], K[:, :, 24:], V[:, :, 24:], chunk=8, initial_state=S0)
    assert orc.rel_err(second, full[:, :, 24:]) < 1e-13
    gf = orc.chunked_backward(Q, K, V, G, chunk=8)
    _, R1 = orc.local_states(Q[:, :, 24:], K[:, :, 24:], V[:, :, 24:], G[:, :, 24:])
    first = orc.chunked_backward(Q[:, :, :24], K[:, :, :24], V[:, :, :24], G[:, :, :24], chunk=8,
                                 final_grad_state=R1)
    last = orc.chunked_backward(Q[:, :, 24:], K[:, :, 24:], V[:, :, 24:], G[:, :, 24:], chunk=8,
                                initial_state=S0)
    for a, b, c in zip(first, last, gf):
        assert orc.rel_err(torch.cat([a, b], dim=2), c) < 1e-13


def test_recurrent_step_oracle_vs_reference(golden):
    """The fp64 restatement of the recurrent step against the reference module's outputs and
    states (from an empty and from a given state), and the reference's own property that the
    steps reproduce the batch layer (test_linear_attention.py:54-79, bound 1e-5)."""
    g = golden("recurrent")
    q, k, v = (T(g[n]) for n in "qkv")
    L = q.shape[1]
    for tag, state in (("empty", None), ("given", [T(g["S0"]), T(g["z0"])])):
        ys = []
        for i in range(L):
            y, state = orc.recurrent_step(q[:, i], k[:, i], v[:, i], state)
            ys.append(y)
        assert (torch.stack(ys, 1) - T(g[tag + "_y"])).abs().max() < 1e-5
        assert orc.rel_err(state[0], T(g[tag + "_S"])) < 1e-6
        assert orc.rel_err(state[1], T(g[tag + "_z"])) < 1e-6
    assert (orc.layer_forward(q, k, v) - T(g["batch_y"])).abs().max() < 1e-5
    assert (T(g["empty_y"]) - T(g["batch_y"])).abs().max() < 1e-5


def test_unmasked_layer_restatement_matches_reference_golden(golden):
    """The oracle's restatement of the unmasked LinearAttention against the reference's own
    output (fixture generated from the unmodified reference module)."""
    g = golden("linear")
    q, k, v = (torch.from_numpy(g[n]) for n in "qkv")
    klen = torch.from_numpy(g["klen"])
    want = orc.linear_layer_forward(q, k, v, key_lengths=klen)
    assert (want - torch.from_numpy(g["y"]).double()).abs().max() < 1e-5
    # the recurrent cross-attention steps of the reference reproduce its batch form
    assert np.abs(g["step_y"] - g["y"]).max() < 1e-5


@pytest.mark.parametrize("D,M", workloads.WIDE_GOLDEN_SHAPES)
def test_wide_shapes_oracle_vs_reference(golden, D, M):
    """Query / value widths that are multiples of 64 above 64 (the shapes the wide tensor-core scans
    take): the sequential C port reproduces the reference's kernel bit for bit, the fp64 blocked
    form agrees with it to fp32 accuracy, on the sampled rows and on the checksums."""
    g = golden("product_wide")
    Q, K, V, G = workloads.wide_golden_inputs(D, M)
    rows = workloads.WIDE_GOLDEN_ROWS
    port = (orc.c_forward(Q, K, V),) + tuple(orc.c_backward(Q, K, V, G))
    f64 = (orc.chunked_forward(Q, K, V, chunk=64),) + tuple(orc.chunked_backward(Q, K, V, G, chunk=64))
    for name, c, x in zip(("out", "gQ", "gK", "gV"), port, f64):
        ref = T(g["%s_%d_%d" % (name, D, M)])
        assert torch.equal(c[:, :, rows], ref), name
        assert orc.rel_err(ref, x[:, :, rows]) < 2e-6, name
        np.testing.assert_allclose(x.sum().item(), g["sum_%s_%d_%d" % (name, D, M)], rtol=1e-5, atol=1e-3)
