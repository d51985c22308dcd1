"""Second opinion on parity: the unmodified reference CUDA kernel (built from the reference checkout into
oracle/_ref by oracle/build_ref.py) on the same inputs. The two kernels sum in different orders, so they agree within
FP32 rounding, not bitwise; both must sit inside the reference's own 2e-5 bound around the FP64 oracle. Skipped when
the reference library was never built."""
import ctypes

import pytest
import torch

from oracle import build_ref
from oracle import decode_gemv_oracle as oc
from oracle import workloads as wl
from tests import helpers as h

pytestmark = pytest.mark.gpu
dev = torch.device("cuda")


@pytest.fixture(scope="module")
def ref():
    lib = build_ref.load()
    if lib is None:
        pytest.skip("oracle/_ref/libdecode_gemv_ref.so was not built")
    return lib


def ref_run(lib, fmt, x, t, out):
    p = lambda a: ctypes.c_void_p(a.data_ptr()) if a is not None else None
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    m, k = x.shape
    n = t[0].shape[0]
    kind = 0 if out.dtype == torch.float32 else 1
    if fmt == "nvfp4":
        code = lib.ref_enqueue_nvfp4(p(x), x.stride(0), 1, p(t[0]), p(t[1]), 0, p(t[2]), p(out), out.stride(0), kind, m,
                                     n, k, stream)
    elif fmt == "bf16":
        code = lib.ref_enqueue_bf16(p(x), x.stride(0), p(t[0]), p(out), out.stride(0), kind, m, n, k, stream)
    else:
        mx = fmt == "mxfp8"
        code = lib.ref_enqueue_fp8(p(x), x.stride(0), 1, p(t[0]), None if mx else p(t[1]), p(t[1]) if mx else None,
                                   p(out), out.stride(0), kind, m, n, k, stream)
    assert code == 0
    return out


@pytest.mark.parametrize("fmt,n,k", [("nvfp4", 1000, 5120), ("fp8", 1024, 5120), ("mxfp8", 1024, 5120),
                                     ("bf16", 1000, 2048)])
def test_reference_kernel_and_ours_agree_within_fp32_rounding(ref, fmt, n, k):
    assert ref.ref_hardware_decode() == 1          # the reference takes its sm_100a path here
    host = {"nvfp4": lambda: wl.ref_nvfp4(n, k), "fp8": lambda: wl.ref_fp8(n, k, False),
            "mxfp8": lambda: wl.ref_fp8(n, k, True), "bf16": lambda: (wl.ref_bf16(n, k),)}[fmt]()
    t = tuple(a.to(dev) for a in host)
    x = wl.activations(16, k).to(dev)
    ours = h.run(fmt, x, t, torch.empty(16, n, device=dev))
    theirs = ref_run(ref, fmt, x, t, torch.empty(16, n, device=dev))
    torch.cuda.synchronize()
    values = oc.values_of(fmt, host)
    assert oc.within_fp32_bound(theirs, x, values)       # the oracle is inside the reference's bound of the reference
    assert oc.within_fp32_bound(ours, x, values)
    assert float((ours - theirs).abs().max() / theirs.abs().max()) < 1e-5
