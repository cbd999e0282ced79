"""What a sequence-parallel rank sees when a peer never delivers -- on ONE GPU, without another
process: ``ftb_exchange_receive`` for rank 1 of a world of two, with nobody playing rank 0.  The
kernel's wait is bounded; with the limit set to a few tens of milliseconds it runs out, the kernel
fills its result with NaN, records ``FTB_ERR_TIMEOUT`` in the device status word and returns, and
the context stays usable.  Nothing here faults or hangs the device: the wait simply ends."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

import fast_transformers_b200 as ftb  # noqa: E402
from fast_transformers_b200 import _native  # noqa: E402


def test_receive_without_a_pusher_gives_up_and_reports(native_lib):
    lib = native_lib
    assert torch.cuda.is_available()
    torch.cuda.synchronize()
    assert lib.ftb_device_status(1) == 0
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    elems = 4096
    buf = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(_native.EXCHANGE_HANDLE_BYTES)
    previous = lib.ftb_exchange_wait_limit_ms(40)
    assert previous == 1000
    _native.check(lib.ftb_exchange_create(2, elems, ctypes.byref(buf), handle), "create")
    try:
        # rank 0 of two has nobody before it: its receive must not wait at all and yields zeros
        first = torch.full((elems,), 3.0, device="cuda")
        _native.check(lib.ftb_exchange_receive(buf, first.data_ptr(), elems, 0, 2, 0, stream), "receive")
        torch.cuda.synchronize()
        assert torch.all(first == 0) and lib.ftb_device_status(0) == 0
        # rank 1 waits for rank 0's state, which never comes
        out = torch.zeros(elems, device="cuda")
        t0 = time.perf_counter()
        _native.check(lib.ftb_exchange_receive(buf, out.data_ptr(), elems, 1, 2, 0, stream), "receive")
        with pytest.raises(_native.NativeError) as e:
            ftb.check_device_status()           # synchronises, raises, clears the word
        waited = time.perf_counter() - t0
        assert e.value.status == _native.ERR_TIMEOUT
        assert 0.02 < waited < 5.0, waited
        assert torch.isnan(out).all()
        # cleared, and the device still computes
        assert lib.ftb_device_status(0) == 0
        assert float((torch.ones(1000, device="cuda") * 2).sum()) == 2000.0
    finally:
        lib.ftb_exchange_wait_limit_ms(previous)
        torch.cuda.synchronize()
        lib.ftb_exchange_destroy(buf)
    assert lib.ftb_exchange_wait_limit_ms(0) == 1000
