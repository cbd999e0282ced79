"""The allocation-free forward entry point, called through the C ABI.

Some users of the library cannot allocate device memory when the product runs (a frozen
allocator in a serving loop, a plugin host that forbids it).  ``ftb_causal_dot_product_static``
keeps its scratch in a static array inside the library; this file checks that it returns what the
ordinary entry point returns, twice in a row (the second call meets the first call's leftovers in
the shared array), that it refuses problems beyond its built-in limit, and that no device memory
is taken while it runs, from torch's pool or from the driver.  The file name sorts last so a run that stops at the
first failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

from fast_transformers_b200 import _native, workloads  # noqa: E402
from fast_transformers_b200.causal_product import causal_dot_product_cuda  # noqa: E402


def _call_static(lib, Q, K, V, out, mode):
    s = _native.strides3
    return lib.ftb_causal_dot_product_static(
        Q.data_ptr(), K.data_ptr(), V.data_ptr(), out.data_ptr(), *Q.shape, V.shape[3],
        s(Q), s(K), s(V), s(out), _native.F32, _native.MODE_IDS[mode],
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("mode", ["mma", "fp32"])
def test_static_scratch_entry_matches_ordinary_entry_twice(native_lib, mode):
    assert torch.cuda.is_available()
    # several segments per head, so the scratch really is used
    Q, K, V, _ = (t.cuda() for t in workloads.make_inputs(2, scale_N=2))
    N, H, L, D = Q.shape
    need = native_lib.ftb_causal_workspace_bytes(N, H, L, D, V.shape[3], _native.F32,
                                                 _native.MODE_IDS[mode], 0, 0)
    assert 0 < need <= _native.STATIC_SCRATCH_BYTES
    want = torch.empty_like(V)
    causal_dot_product_cuda(Q, K, V, want, mode)
    # a different problem first, to leave foreign data in the shared array
    Q2, K2, V2 = (t.flip(2).contiguous() for t in (Q, K, V))
    want2 = torch.empty_like(V2)
    causal_dot_product_cuda(Q2, K2, V2, want2, mode)
    torch.cuda.synchronize()

    got2, got, again = (torch.full_like(V, float("nan")) for _ in range(3))
    # torch's counter sees what is taken from torch's pool; the driver's free-memory figure also
    # sees a raw cudaMalloc made inside the library (the same kernels have already run above, so
    # no module is loaded for the first time in between)
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    assert _call_static(native_lib, Q2, K2, V2, got2, mode) == _native.OK
    assert _call_static(native_lib, Q, K, V, got, mode) == _native.OK
    assert _call_static(native_lib, Q, K, V, again, mode) == _native.OK
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] >= free_before
    # same kernels, same order of operations: the results are identical, not merely close
    assert torch.equal(got2, want2)
    assert torch.equal(got, want)
    assert torch.equal(again, want)
    assert native_lib.ftb_device_status(0) == 0


def test_static_scratch_entry_rejects_problems_beyond_its_limit(native_lib):
    x = torch.zeros(1, 1, 4, 64, device="cuda")
    out = torch.full_like(x, 7.0)
    s = _native.strides3(x)
    # shape arguments describe one head of a million positions with 512 x 512 states: hundreds of
    # segments of 1 MiB each, far beyond 16 MiB; the call must refuse before touching any pointer
    st = native_lib.ftb_causal_dot_product_static(
        x.data_ptr(), x.data_ptr(), x.data_ptr(), out.data_ptr(), 1, 1, 1 << 20, 512, 512,
        s, s, s, s, _native.F32, _native.MODE_FP32_SIMT,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert st == _native.ERR_STATIC_LIMIT
    assert b"static" in native_lib.ftb_status_string(st)
    torch.cuda.synchronize()
    assert torch.all(out == 7.0)
