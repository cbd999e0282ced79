"""ctypes binding of ``libftb200.so`` (the C ABI declared in ``include/ftb200.h``).

The library is looked up next to this file.  It is never rebuilt or replaced silently at
call time: if it is missing, ``lib()`` raises ``RuntimeError`` telling how to build it
(``python fast-transformers_b200/build.py``).  There is no other implementation to fall
back to.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FTB200_LIB") or os.path.join(_HERE, "libftb200.so")

OK, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_WORKSPACE, ERR_CUDA, ERR_TIMEOUT, ERR_INVALID, \
    ERR_STATIC_LIMIT = range(8)
STATIC_SCRATCH_BYTES = 16 * 1024 * 1024
F32, BF16 = 0, 1
MODE_FP32_SIMT, MODE_MMA, MODE_MMA_X3 = 0, 1, 2
MODE_IDS = {"fp32": MODE_FP32_SIMT, "mma": MODE_MMA, "tf32x3": MODE_MMA_X3}

# every symbol include/ftb200.h declares
EXPORTS = (
    "ftb_version", "ftb_status_string", "ftb_last_cuda_error", "ftb_causal_workspace_bytes",
    "ftb_causal_dot_product", "ftb_causal_dot_backward", "ftb_causal_state_sum",
    "ftb_launch_count", "ftb_timing_enable", "ftb_timing_read", "ftb_device_status",
    "ftb_causal_dot_product_static", "ftb_recurrent_linear_step",
    "ftb_causal_normaliser_workspace_bytes", "ftb_causal_normaliser", "ftb_causal_normaliser_backward",
    "ftb_elu_feature_map", "ftb_elu_feature_map_backward",
    "ftb_exchange_bytes", "ftb_exchange_create", "ftb_exchange_open", "ftb_exchange_close",
    "ftb_exchange_destroy", "ftb_exchange_push", "ftb_exchange_receive",
    "ftb_exchange_wait_limit_ms", "ftb_exchange_push_parts", "ftb_causal_state_parts",
    "ftb_linear_apply_state", "ftb_favor_feature_map", "ftb_recurrent_cross_linear_step",
    "ftb_causal_dot_product_normalised", "ftb_favor_feature_map_backward",
    "ftb_causal_normaliser_backward_add", "ftb_normalised_output_grads",
    "ftb_causal_normaliser_backward_elu",
)
KERNEL_KINDS = ("state_sum", "state_prefix", "simt_scan", "mma_fwd", "mma_bwd", "mma_state",
                "mma_bwd_qr", "mma_bwd_multi", "recurrent_step", "normaliser", "feature_map",
                "rank_exchange", "apply_state")

_lib = None
_i64, _vp, _int, _sz = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_i64p = ctypes.POINTER(ctypes.c_int64)


class NativeError(RuntimeError):
    """A non-zero status returned by the native library."""

    def __init__(self, status, message):
        super().__init__(message)
        self.status = status


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "native library %s not found; build it with `python fast-transformers_b200/build.py` "
            "(needs nvcc 12.9). There is no fallback implementation." % LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    L.ftb_version.restype = _int
    L.ftb_status_string.restype = ctypes.c_char_p
    L.ftb_status_string.argtypes = [_int]
    L.ftb_last_cuda_error.restype = _int
    L.ftb_causal_workspace_bytes.restype = _sz
    L.ftb_causal_workspace_bytes.argtypes = [_i64] * 5 + [_int] * 4
    L.ftb_causal_dot_product.restype = _int
    L.ftb_causal_dot_product.argtypes = (
        [_vp] * 4 + [_i64] * 5 + [_i64p] * 4 + [_int, _int, _vp, _vp, _int, _vp, _sz, _vp])
    L.ftb_causal_dot_product_normalised.restype = _int
    L.ftb_causal_dot_product_normalised.argtypes = (
        [_vp] * 5 + [_i64] * 5 + [_i64p] * 5 + [_int, _int, ctypes.c_float, _vp, _sz, _vp])
    L.ftb_causal_dot_backward.restype = _int
    L.ftb_causal_dot_backward.argtypes = (
        [_vp] * 7 + [_i64] * 5 + [_i64p] * 7 + [_int, _int, _vp, _vp, _vp, _int, _vp, _sz, _vp])
    L.ftb_causal_state_sum.restype = _int
    L.ftb_causal_state_sum.argtypes = (
        [_vp] * 3 + [_i64] * 5 + [_i64p] * 2 + [_int, _int, _int, _vp, _sz, _vp])
    L.ftb_causal_dot_product_static.restype = _int
    L.ftb_causal_dot_product_static.argtypes = (
        [_vp] * 4 + [_i64] * 5 + [_i64p] * 4 + [_int, _int, _vp])
    L.ftb_recurrent_linear_step.restype = _int
    L.ftb_recurrent_linear_step.argtypes = (
        [_vp] * 6 + [_i64] * 4 + [_i64p] * 4 + [_int, _int, ctypes.c_float, _vp])
    L.ftb_causal_normaliser_workspace_bytes.restype = _sz
    L.ftb_causal_normaliser_workspace_bytes.argtypes = [_i64] * 4 + [_int]
    L.ftb_causal_normaliser.restype = _int
    L.ftb_causal_normaliser.argtypes = [_vp] * 3 + [_i64] * 4 + [_i64p] * 3 + [_int, _vp, _sz, _vp]
    L.ftb_causal_normaliser_backward.restype = _int
    L.ftb_causal_normaliser_backward.argtypes = (
        [_vp] * 5 + [_i64] * 4 + [_i64p] * 5 + [_int, _vp, _sz, _vp])
    L.ftb_causal_normaliser_backward_elu.restype = _int
    L.ftb_causal_normaliser_backward_elu.argtypes = (
        [_vp] * 8 + [_i64] * 4 + [_i64p] * 7 + [_int, _vp, _sz, _vp])
    L.ftb_normalised_output_grads.restype = _int
    L.ftb_normalised_output_grads.argtypes = [_vp] * 5 + [_i64, _i64, ctypes.c_float, _vp]
    L.ftb_causal_normaliser_backward_add.restype = _int
    L.ftb_causal_normaliser_backward_add.argtypes = L.ftb_causal_normaliser_backward.argtypes
    L.ftb_elu_feature_map.restype = _int
    L.ftb_elu_feature_map.argtypes = [_vp, _vp, _vp, _i64, _i64, _int, _vp]
    L.ftb_elu_feature_map_backward.restype = _int
    L.ftb_elu_feature_map_backward.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp]
    L.ftb_exchange_bytes.restype = _sz
    L.ftb_exchange_bytes.argtypes = [_int, _i64]
    L.ftb_exchange_create.restype = _int
    L.ftb_exchange_create.argtypes = [_int, _i64, ctypes.POINTER(_vp), ctypes.c_char_p]
    L.ftb_exchange_open.restype = _int
    L.ftb_exchange_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(_vp)]
    L.ftb_exchange_close.restype = _int
    L.ftb_exchange_close.argtypes = [_vp]
    L.ftb_exchange_destroy.restype = _int
    L.ftb_exchange_destroy.argtypes = [_vp]
    L.ftb_exchange_push.restype = _int
    L.ftb_exchange_push.argtypes = [_vp, _i64, ctypes.POINTER(_vp), _int, _int, _int, _vp]
    L.ftb_exchange_push_parts.restype = _int
    L.ftb_exchange_push_parts.argtypes = [_vp, _i64, _int, _i64, ctypes.POINTER(_vp), _int, _int, _int, _vp]
    L.ftb_causal_state_parts.restype = _int
    L.ftb_causal_state_parts.argtypes = [_i64] * 5 + [_int, _int]
    L.ftb_exchange_receive.restype = _int
    L.ftb_exchange_receive.argtypes = [_vp, _vp, _i64, _int, _int, _int, _vp]
    L.ftb_linear_apply_state.restype = _int
    L.ftb_linear_apply_state.argtypes = [_vp] * 3 + [_i64] * 5 + [_i64p] * 2 + [_int, _int, _int, _vp]
    L.ftb_recurrent_cross_linear_step.restype = _int
    L.ftb_recurrent_cross_linear_step.argtypes = (
        [_vp] * 4 + [_i64] * 4 + [_i64p] * 2 + [_int, _int, ctypes.c_float, _vp])
    L.ftb_favor_feature_map_backward.restype = _int
    L.ftb_favor_feature_map_backward.argtypes = [_vp] * 5 + [_i64] * 7 + [ctypes.c_float, _vp]
    L.ftb_favor_feature_map.restype = _int
    L.ftb_favor_feature_map.argtypes = [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, ctypes.c_float, _vp]
    L.ftb_exchange_wait_limit_ms.restype = _int
    L.ftb_exchange_wait_limit_ms.argtypes = [_int]
    L.ftb_launch_count.restype = ctypes.c_uint64
    L.ftb_device_status.restype = _int
    L.ftb_device_status.argtypes = [_int]
    L.ftb_timing_enable.restype = None
    L.ftb_timing_enable.argtypes = [_int]
    L.ftb_timing_read.restype = _int
    L.ftb_timing_read.argtypes = [ctypes.POINTER(ctypes.c_float), ctypes.POINTER(_int), _int]
    _lib = L
    return L


def timing_read():
    """{kernel kind: (milliseconds, launches)} recorded since ``ftb_timing_enable(1)``."""
    n = len(KERNEL_KINDS)
    ms = (ctypes.c_float * n)()
    cnt = (_int * n)()
    check(lib().ftb_timing_read(ms, cnt, n), "ftb_timing_read")
    return {KERNEL_KINDS[i]: (ms[i], cnt[i]) for i in range(n) if cnt[i]}


FEATURE_NONE, FEATURE_ELU1 = 0, 1
EXCHANGE_HANDLE_BYTES = 64


def strides2(t):
    s = t.stride()
    return (ctypes.c_int64 * 2)(s[0], s[1])


def strides3(t):
    s = t.stride()
    return (ctypes.c_int64 * 3)(s[0], s[1], s[2])


def check(status, what):
    if status == OK:
        return
    L = lib()
    msg = L.ftb_status_string(status).decode()
    if status == ERR_CUDA:
        msg += " (cudaError %d)" % L.ftb_last_cuda_error()
    raise NativeError(status, "%s failed: %s" % (what, msg))
