"""Calls into the C ABI with torch tensors (device pointers, current stream), for the GPU tests."""
import ctypes

import torch

from crit_kernels_b200 import cabi


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _kind(out):
    return 0 if out.dtype == torch.float32 else 1


def abi_nvfp4(x, codes, scales, inverse, out, blocked=False):
    m, k = x.shape
    return cabi.load().dg_enqueue_nvfp4(_ptr(x), x.stride(0), int(x.dtype == torch.bfloat16), _ptr(codes),
                                        _ptr(scales), int(blocked), _ptr(inverse), _ptr(out), out.stride(0),
                                        _kind(out), m, codes.shape[0], k, _stream())


def abi_fp8(x, codes, scales, out):
    m, k = x.shape
    mx = scales.dtype == torch.uint8
    return cabi.load().dg_enqueue_fp8(_ptr(x), x.stride(0), int(x.dtype == torch.bfloat16), _ptr(codes),
                                      None if mx else _ptr(scales), _ptr(scales) if mx else None, _ptr(out),
                                      out.stride(0), _kind(out), m, codes.shape[0], k, _stream())


def abi_bf16(x, w, out):
    m, k = x.shape
    return cabi.load().dg_enqueue_bf16(_ptr(x), x.stride(0), _ptr(w), _ptr(out), out.stride(0), _kind(out), m,
                                       w.shape[0], k, _stream())


def run(fmt, x, tensors, out, blocked=False):
    """One GEMV of `fmt` through the C ABI; asserts the call was accepted; returns out."""
    if fmt == "nvfp4":
        code = abi_nvfp4(x, *tensors, out, blocked=blocked)
    elif fmt in ("fp8", "mxfp8"):
        code = abi_fp8(x, *tensors, out)
    else:
        code = abi_bf16(x, *tensors, out)
    assert code == 0, f"{fmt}: cudaError {code}"
    return out
