"""ctypes view of the C ABI (include/decode_gemv_b200.h), for tests, benches and callers without torch ops.

Loads lib/libdecode_gemv_b200.so; there is no fallback when it is missing."""
from __future__ import annotations

import ctypes
import os

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libdecode_gemv_b200.so")

_p, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int)
SIGNATURES = {
    "dg_enqueue_nvfp4": (_i, [_p, _i, _i, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _p]),
    "dg_enqueue_nvfp4_allgather": (_i, [_p, _i, _i, _p, _p, _i, _p, ctypes.POINTER(_p), ctypes.POINTER(_p), _i, _i, _i,
                                        _i, _i, _i, _i, _p]),
    "dg_enqueue_nvfp4_allgather_noalloc": (_i, [_p, _i, _i, _p, _p, _i, _p, ctypes.POINTER(_p), _f, _i, _i, _i, _i, _i, _i,
                                                _i, _i, _p]),
    "dg_enqueue_gather_wait": (_i, [_p, _i, ctypes.c_uint, _p]),
    "dg_enqueue_swiglu": (_i, [_p, ctypes.c_longlong, _i, _i, _i, _p, ctypes.c_longlong, _i, _p]),
    "dg_enqueue_nvfp4_gate_up_swiglu": (_i, [_p, _i, _i, _p, _p, _i, _p, _p, _i, _i, _i, _i, _i, _p]),
    "dg_batch_blob_bytes": (ctypes.c_ulonglong, [_i]),
    "dg_encode_nvfp4_batch": (_i, [_p, _i, _i, _i, _i, _i, _i, ctypes.POINTER(_p), _i, _p, _p]),
    "dg_enqueue_batch": (_i, [_p, _p]),
    "dg_enqueue_fp8": (_i, [_p, _i, _i, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "dg_enqueue_bf16": (_i, [_p, _i, _p, _p, _i, _i, _i, _i, _i, _p]),
    "dg_enqueue_dequantize": (_i, [_p, _p, _p, _p, _i, _i, _i, _p]),
    "dg_enqueue_quantize_fp8_rows": (_i, [_p, ctypes.c_longlong, _i, _i, _p, ctypes.c_longlong, _p, _p]),
    "dg_enqueue_quantize_nvfp4": (_i, [_p, ctypes.c_longlong, _i, _i, ctypes.c_float, ctypes.c_float, _p, _p, _p]),
    "dg_hardware_decode": (_i, []),
    "dg_plan": (_i, [_i, _i, _i, _i, _f]),
    "dg_take_status": (_i, []),
    "dg_set_static_weights": (_i, [_i]),
    "dg_set_trace": (_i, [_p, _i]),
    "dg_reset_counters": (_i, [_p, _p]),
    "dg_reset_noalloc_channel": (_i, [_i, _p]),
    "dg_set_wait_limit_ns": (ctypes.c_ulonglong, [ctypes.c_ulonglong]),
    "dg_version": (_i, []),
}


class Nvfp4BatchItem(ctypes.Structure):
    """DgNvfp4BatchItem of include/decode_gemv_b200.h."""
    _fields_ = [("x", _p), ("codes", _p), ("scales", _p), ("inverse", _p), ("out", _p), ("peer_out", ctypes.POINTER(_p)),
                ("ldx", _i), ("ldo", _i), ("blocked", _i), ("N", _i), ("K", _i)]


FMT = {"bf16": 0, "fp8": 1, "mxfp8": 2, "nvfp4": 3}
_lib = None


def library_path() -> str:
    return _PATH


def load() -> ctypes.CDLL:
    """The loaded library with argument types set; raises OSError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            raise OSError(f"{_PATH} is missing: build it with `python -m crit_kernels_b200.builder`")
        lib = ctypes.CDLL(_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def plan(fmt: str, m: int, n: int, k: int) -> dict:
    """The launch shape a call of these sizes gets (host only)."""
    out = (ctypes.c_int * 6)()
    code = load().dg_plan(FMT[fmt], m, n, k, out)
    if code:
        raise ValueError(f"dg_plan refused fmt={fmt} M={m} N={n} K={k} (cudaError {code})")
    keys = ("ctas", "rows_per_warp", "steps", "stages", "stage_bytes", "smem_bytes")
    return dict(zip(keys, out))
