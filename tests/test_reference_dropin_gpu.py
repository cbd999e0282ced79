"""The drop-in boundary exercised with the REFERENCE's own classes.

The reference dispatches its causal product through two class-level tables keyed by device type
(``fast_transformers/causal_product/__init__.py:23-30``); without its CUDA extension the
``"cuda"`` entries are ``None`` (``:12-17``).  This test imports the unmodified reference package
(an offline install under ``baseline/_ref``: its Python modules and its CPU extensions, no CUDA
extension), assigns this library's two native functions to those entries -- the two lines a
maintainer of the reference would add -- and then runs the reference's ``CausalDotProduct`` and
its ``CausalLinearAttention`` (with the reference's masks, feature map and registry untouched)
on CUDA tensors, against the golden outputs that the same reference produced on the CPU.

Skipped when no install of the reference is present (the checkout itself is not read here).
"""
import importlib
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def T(a):
    return torch.from_numpy(np.asarray(a))


@pytest.fixture(scope="module")
def reference(native_lib):
    if not os.path.isdir(os.path.join(REF, "fast_transformers")):
        pytest.skip("no install of the reference under baseline/_ref")
    assert torch.cuda.is_available()
    import fast_transformers_b200 as ftb
    from fast_transformers_b200.causal_product import (causal_dot_backward_cuda,
                                                       causal_dot_product_cuda)
    sys.path.insert(0, REF)
    try:
        cp = importlib.import_module("fast_transformers.causal_product")
        cla = importlib.import_module("fast_transformers.attention.causal_linear_attention")
        masking = importlib.import_module("fast_transformers.masking")
    finally:
        sys.path.remove(REF)
    assert os.path.realpath(cp.__file__).startswith(os.path.realpath(REF))
    table, table_b = cp.CausalDotProduct.dot, cp.CausalDotProduct.dot_backward
    saved = (table.get("cuda"), table_b.get("cuda"), ftb.get_mode())
    assert saved[0] is None, "the reference's CUDA extension is not part of this install"
    # ---- the binding: two assignments --------------------------------------------------
    table["cuda"] = causal_dot_product_cuda            # (Q, K, V, product) -> None
    table_b["cuda"] = causal_dot_backward_cuda         # (Q, K, V, grad_out, gQ, gK, gV) -> None
    yield cp, cla, masking, ftb
    table["cuda"], table_b["cuda"] = saved[0], saved[1]
    ftb.set_mode(saved[2])
    torch.cuda.synchronize()
    assert native_lib.ftb_device_status(1) == 0


@pytest.mark.parametrize("mode,tol", [("fp32", 1e-5), ("mma", 2e-2)])
def test_reference_autograd_function_runs_on_this_library(reference, golden, mode, tol):
    """``fast_transformers.causal_product.causal_dot_product`` on CUDA tensors: the reference's
    Function allocates zeroed outputs, passes ``.data`` views and ``grad_out`` untouched
    (``__init__.py:41-49,59-72``); the results are compared with what its own CPU kernel gave."""
    cp, _, _, ftb = reference
    from oracle import causal_oracle as orc
    from fast_transformers_b200 import workloads
    g = golden("product_config1_sample")
    Q, K, V, G = workloads.make_inputs(1)
    q, k, v = (t.cuda().requires_grad_(True) for t in (Q, K, V))
    launches = ftb._native.lib().ftb_launch_count()
    ftb.set_mode(mode)      # process-wide: the backward runs on an autograd thread
    out = cp.causal_dot_product(q, k, v)
    out.backward(G.cuda())
    torch.cuda.synchronize()
    assert ftb._native.lib().ftb_launch_count() > launches, "this library's kernels did not run"
    rows = T(g["rows"])
    for name, a in zip(("out", "gQ", "gK", "gV"), (out, q.grad, k.grad, v.grad)):
        assert a.is_cuda and a.dtype == torch.float32
        assert orc.rel_err(a.detach().cpu()[:, :, rows], T(g[name])) < tol, name


@pytest.mark.parametrize("case", ["eq", "lt"])
def test_reference_layer_runs_on_this_library(reference, golden, case):
    """The reference's ``CausalLinearAttention.forward`` (``causal_linear_attention.py:71-104``),
    its own masks and feature map, on CUDA: the only code of this repository on the path is the
    pair of native functions behind the two table entries.  Bounds as in the layer test of this
    repository: 5e-4 absolute, the reference's own for the normalised product."""
    _, cla, masking, ftb = reference
    ftb.set_mode("fp32")
    g = golden("layer")
    q, k, v, w = (T(g[case + "_" + n]).cuda() for n in "qkvw")
    klen = T(g[case + "_klen"]).cuda()
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    N, L = q.shape[:2]
    S = k.shape[1]
    att = cla.CausalLinearAttention(q.shape[3])
    y = att(q, k, v, masking.TriangularCausalMask(L, device="cuda"),
            masking.LengthMask(torch.full((N,), L, device="cuda")),
            masking.LengthMask(klen, max_len=S))
    assert (y.cpu() - T(g[case + "_y"])).abs().max() < 5e-4
    (y * w).sum().backward()
    for n, t in (("gq", q), ("gk", k), ("gv", v)):
        assert (t.grad.cpu() - T(g[case + "_" + n])).abs().max() < 5e-4, n


def test_reference_registry_builds_the_layer_on_this_library(reference, golden):
    """``AttentionBuilder`` of the reference with ``attention_type="causal-linear"`` -- the
    registry entry (``causal_linear_attention.py:109-116``) is the reference's own -- gives a
    layer whose product runs here."""
    _, _, masking, ftb = reference
    sys.path.insert(0, REF)
    try:
        builders = importlib.import_module("fast_transformers.builders")
    finally:
        sys.path.remove(REF)
    ftb.set_mode("fp32")
    g = golden("layer")
    att = builders.AttentionBuilder.from_kwargs(query_dimensions=int(g["eq_q"].shape[3])).get("causal-linear")
    q, k, v = (T(g["eq_" + n]).cuda() for n in "qkv")
    N, L = q.shape[:2]
    lm = masking.LengthMask(T(g["eq_klen"]).cuda(), max_len=L)
    y = att(q, k, v, masking.TriangularCausalMask(L, device="cuda"),
            masking.LengthMask(torch.full((N,), L, device="cuda")), lm)
    assert (y.cpu() - T(g["eq_y"])).abs().max() < 5e-4
