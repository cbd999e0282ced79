"""HostStepPipeline: steps with host-resident inputs and results, copies overlapping kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import fast_transformers_b200 as ftb  # noqa: E402
from fast_transformers_b200.causal_product import causal_dot_product  # noqa: E402
from fast_transformers_b200.host_io import HostStepPipeline  # noqa: E402
from oracle import causal_oracle as orc  # noqa: E402


def test_pipeline_matches_step_by_step(native_lib):
    g = torch.Generator().manual_seed(11)
    shape = (2, 2, 300, 32)
    steps = [[torch.rand(shape, generator=g).pin_memory() for _ in range(4)] for _ in range(5)]
    outs = [[torch.empty(shape).pin_memory() for _ in range(4)] for _ in range(5)]

    def compute(q, k, v, grad):
        q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
        with ftb.mode("fp32"):
            out = causal_dot_product(q, k, v)
            out.backward(grad)
        return out.detach(), q.grad, k.grad, v.grad

    pipe = HostStepPipeline(compute, steps[0], device="cuda")
    for hin, hout in zip(steps, outs):
        pipe.run(hin, hout)
    pipe.synchronize()
    for hin, hout in zip(steps, outs):
        Q, K, V, G = hin
        want = (orc.chunked_forward(Q, K, V),) + tuple(orc.chunked_backward(Q, K, V, G))
        for a, b in zip(hout, want):
            assert orc.rel_err(a, b) < 1e-5
    assert native_lib.ftb_device_status(1) == 0
