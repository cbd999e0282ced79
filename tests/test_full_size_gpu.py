"""Parity at the benchmark's own sizes: configurations 2, 4 and 5 run at full size on the GPU
(every (batch, head) pair), and the output and all three gradients of sampled pairs are compared
with the fp64 blocked recurrence (``oracle.chunked_forward`` / ``chunked_backward``, the dense form
of the reference's tests regrouped, ``tests/causal_product/test_causal_product_cpu.py:45-47,63-70``).

Tolerances on ``max|x - x64| / max|x64|`` (the maximum taken over the sampled pairs):
1e-5 for the ``"fp32"`` mode and for ``"tf32x3"`` (split TF32 operands, three products each), 2e-2
for the ``"mma"`` mode (TF32 or bf16 operands, fp32 accumulation and state).  The measured errors go to the file named by ``FTB200_PARITY_LOG`` (one
JSON object per line) when that variable is set.
"""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import causal_oracle as orc  # noqa: E402
from fast_transformers_b200 import workloads  # noqa: E402
import fast_transformers_b200 as ftb  # noqa: E402
from fast_transformers_b200.causal_product import causal_dot_product  # noqa: E402

NAMES = ("out", "gQ", "gK", "gV")
TOL = {"fp32": 1e-5, "mma": 2e-2, "tf32x3": 1e-5}


@pytest.fixture(scope="module", autouse=True)
def _lib(native_lib):
    assert torch.cuda.is_available()
    yield native_lib
    torch.cuda.synchronize()
    assert native_lib.ftb_device_status(1) == 0, "a kernel recorded a device-side error"


def _run(Q, K, V, G, mode):
    q, k, v = (t.cuda().requires_grad_(True) for t in (Q, K, V))
    with ftb.mode(mode):
        out = causal_dot_product(q, k, v)
        out.backward(G.cuda())
    torch.cuda.synchronize()
    return out.detach(), q.grad, k.grad, v.grad


def _check_pairs(config, mode, inputs, got, pairs, chunk=256):
    """Compare the (n, h) pairs in ``pairs`` with the fp64 oracle; returns the errors."""
    Q, K, V, G = inputs
    errs = dict.fromkeys(NAMES, 0.0)
    for n, h in pairs:
        sub = [t[n:n + 1, h:h + 1].float() for t in (Q, K, V, G)]
        want = (orc.chunked_forward(*sub[:3], chunk=chunk),) + tuple(
            orc.chunked_backward(*sub, chunk=chunk))
        for name, a, b in zip(NAMES, got, want):
            assert a.dtype == Q.dtype
            errs[name] = max(errs[name], orc.rel_err(a[n:n + 1, h:h + 1], b))
    line = {"config": config, "mode": mode, "dtype": str(Q.dtype).replace("torch.", ""),
            "shape": list(Q.shape) + [V.shape[3]], "pairs": [list(p) for p in pairs], "rel_err": errs,
            "tolerance": TOL[mode]}
    print("PARITY " + json.dumps(line))
    log = os.environ.get("FTB200_PARITY_LOG")
    if log:
        with open(log, "a") as f:
            f.write(json.dumps(line) + "\n")
    for name in NAMES:
        assert errs[name] < TOL[mode], "config %d %s %s: rel err %.3e" % (config, mode, name, errs[name])
    return errs


@pytest.mark.parametrize("mode", ["mma", "fp32", "tf32x3"])
def test_config2_full_size_all_pairs(mode):
    """The benchmarked workload (N8 H8 L4096 D=M=64 fp32): every one of the 64 pairs, output and
    gradients."""
    inputs = workloads.make_inputs(2)
    got = _run(*inputs, mode)
    N, H = inputs[0].shape[:2]
    _check_pairs(2, mode, inputs, got, [(n, h) for n in range(N) for h in range(H)])


def test_config4_full_length_bf16():
    """One sequence of 262 144 positions, 16 heads, D = M = 128, bf16 tensors and fp32 state: 228
    chunks per segment with positive features, so the state entries grow with the position and
    every chunk rounds them to bf16 as an operand.  Two of the 16 heads through the oracle."""
    inputs = workloads.make_inputs(4)
    assert inputs[0].shape == (1, 16, 262144, 128) and inputs[0].dtype == torch.bfloat16
    got = _run(*inputs, "mma")
    _check_pairs(4, "mma", inputs, got, [(0, 0), (0, 11)], chunk=512)


@pytest.mark.parametrize("mode", ["mma", "fp32"])
def test_config5_full_size_favor_features(mode):
    """Favor features (D = 256 of a 64-wide query, M = 64) at N4 H12 L16384; two pairs."""
    inputs = workloads.make_inputs(5)
    assert inputs[0].shape == (4, 12, 16384, 256) and inputs[2].shape[3] == 64
    got = _run(*inputs, mode)
    _check_pairs(5, mode, inputs, got, [(0, 0), (3, 7)])
