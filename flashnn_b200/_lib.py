"""ctypes binding of the C ABI declared in include/flashnn_b200.h.

Loading never falls back to anything: if the shared library is absent, or the
process has no CUDA device, the operators raise.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashnn_b200.so")

F16, BF16, F32 = 0, 1, 2

# every symbol include/flashnn_b200.h declares: name -> (restype, argtypes)
_c = ctypes
SIGNATURES = {
    "fnn_version": (_c.c_int, []),
    "fnn_last_error_string": (_c.c_char_p, []),
    "fnn_status_string": (_c.c_char_p, [_c.c_int]),
    "fnn_device_status": (_c.c_int, [_c.POINTER(_c.c_int)]),
    "fnn_dynamic_quant": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64,
                                     _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p]),
    "fnn_gemm_a8w8": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int64,
                                 _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int,
                                 _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                                 _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "fnn_gemm_a8w8_workspace_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64, _c.c_int64]),
    "fnn_gemm_a8w8_plan": (_c.c_int, [_c.c_int64, _c.c_int64, _c.c_int64, _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "fnn_gemm_weight_only": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_int,
                                        _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64,
                                        _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int, _c.c_int64,
                                        _c.c_int64, _c.c_int64, _c.c_int64,
                                        _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "fnn_gemm_weight_only_workspace_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64, _c.c_int64,
                                                           _c.c_int, _c.c_int64]),
    "fnn_fused_moe_a8w8": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64,
                                      _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int,
                                      _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int, _c.c_int,
                                      _c.c_int, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "fnn_fused_moe_a8w8_workspace_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64]),
    "fnn_fused_moe_a16w4": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64,
                                       _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_int,
                                       _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int, _c.c_int,
                                       _c.c_int, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p]),
    "fnn_fused_moe_a16w4_ws": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_int64,
                                          _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_int,
                                          _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int, _c.c_int,
                                          _c.c_int, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "fnn_fused_moe_a16w4_workspace_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int]),
    "fnn_set_option": (_c.c_int, [_c.c_int, _c.c_int]),
    "fnn_get_option": (_c.c_int, [_c.c_int]),
    "fnn_rms_norm_dquant": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_int,
                                       _c.c_float, _c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_void_p]),
    "fnn_layer_norm_dquant": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p,
                                         _c.c_void_p, _c.c_int, _c.c_float, _c.c_void_p, _c.c_int64, _c.c_void_p,
                                         _c.c_void_p]),
    "fnn_gemm_weight_only_prefill_static": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_int,
                                                       _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_int,
                                                       _c.c_void_p, _c.c_int, _c.c_int64,
                                                       _c.c_int64, _c.c_int64, _c.c_int64, _c.c_void_p]),
}

_lib = None
_lock = threading.Lock()


class FlashNNError(RuntimeError):
    """A non-zero status from the C ABI: (status code, message)."""

    def __init__(self, status, message):
        super().__init__(status, message)
        self.status = status
        self.message = message

    def __str__(self):
        return f"flashnn_b200 status {self.status}: {self.message}"


def lib():
    """The loaded shared library (loads it on first use)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise FlashNNError(-1, f"{LIB_PATH} is missing: build it with "
                                           "`python -m flashnn_b200.build`; there is no fallback path")
                handle = ctypes.CDLL(LIB_PATH)
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(handle, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def check(status: int):
    if status != 0:
        l = lib()
        raise FlashNNError(status, f"{l.fnn_status_string(status).decode()}: "
                                   f"{l.fnn_last_error_string().decode()}")


OPT_STATIC_WEIGHTS = 1
OPT_TEST_STALL_US = 2  # test hook, see include/flashnn_b200.h
OPT_A8W8_PAIR_TILE = 3  # tuning hook
OPT_A8W8_BALANCED = 4  # 0 by shape, 1 always where possible, 2 never
OPT_A8W8_EPILOGUE_WARPS = 5  # tuning hook: 4 keeps four epilogue warps per CTA for every K


def set_option(option: int, value: int) -> None:
    check(lib().fnn_set_option(option, int(value)))


def device_status() -> int:
    """Synchronises, then returns (and clears) the device status word; raises if a kernel
    gave up on a bounded wait."""
    code = ctypes.c_int(0)
    check(lib().fnn_device_status(ctypes.byref(code)))
    return code.value


def a8w8_plan(m: int, n: int, k: int):
    """(kernel, tile width) fnn_gemm_a8w8 picks for this shape: kernel 0 = single CTA, 1 = CTA pair, 2 = streaming decode,
    3 = CTA pair with the K blocks dealt out evenly (needs the workspace)."""
    kern, tile = ctypes.c_int(0), ctypes.c_int(0)
    check(lib().fnn_gemm_a8w8_plan(m, n, k, ctypes.byref(kern), ctypes.byref(tile)))
    return kern.value, tile.value
