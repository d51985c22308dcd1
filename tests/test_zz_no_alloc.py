"""The entry point for callers that cannot allocate device memory (dg_enqueue_nvfp4_allgather_noalloc): a serving
process whose HBM is fully committed to its own arenas, or a host that forbids cudaMalloc after start-up, still gets
the GEMV with the fused all-gather, because the arrival counters it needs are built into the library instead of being
passed in. Called through the C ABI with one rank on one GPU (peer access is not needed then), twice in a row on the
same channel, and compared bit for bit with the existing entry point that takes caller-allocated counters. The file
sorts last so that a run that stops at the first failure has already run every other test."""
import ctypes

import pytest
import torch

from crit_kernels_b200 import cabi
from oracle import workloads as wl

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def test_built_in_counters_give_the_bits_of_caller_allocated_counters():
    dev = torch.device("cuda")
    lib = cabi.load()
    n, k = 1000, 4096
    codes, scales, inverse = (t.to(dev) for t in wl.cfg_nvfp4(n, k, seed=31))
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    devices = (ctypes.c_int * 1)(torch.cuda.current_device())
    for m in (1, 7, 16):
        x = wl.activations(m, k, seed=40 + m).to(dev)
        # existing entry point: the caller allocates (and zeroes) the block of counters
        want = torch.zeros(1, m, n, dtype=torch.bfloat16, device=dev)
        flags = torch.zeros(4, dtype=torch.int32, device=dev)
        assert lib.dg_enqueue_nvfp4_allgather(_ptr(x), x.stride(0), 1, _ptr(codes), _ptr(scales), 0, _ptr(inverse),
                                              (ctypes.c_void_p * 1)(want.data_ptr()),
                                              (ctypes.c_void_p * 1)(flags.data_ptr()), 1, 0, 0, 1, m, n, k, stream) == 0
        torch.cuda.synchronize()
        # new entry point: nothing allocated for it; two calls in a row on channel 3 (slots 0 then 1)
        for call in range(2):
            found = torch.full((1, m, n), -1.0, dtype=torch.bfloat16, device=dev)   # an output buffer the caller owns
            code = lib.dg_enqueue_nvfp4_allgather_noalloc(_ptr(x), x.stride(0), 1, _ptr(codes), _ptr(scales), 0,
                                                          _ptr(inverse), (ctypes.c_void_p * 1)(found.data_ptr()),
                                                          devices, 1, 0, 3, call & 1, 1, m, n, k, stream)
            assert code == 0, code
            torch.cuda.synchronize()
            assert torch.equal(found.view(torch.int16), want.view(torch.int16)), (m, call)   # bit-exact
    assert lib.dg_take_status() == 0


def test_sizes_beyond_the_built_in_counters_are_refused():
    dev = torch.device("cuda")
    lib = cabi.load()
    n, k, m = 64, 256, 2
    codes, scales, inverse = (t.to(dev) for t in wl.cfg_nvfp4(n, k))
    x = wl.activations(m, k).to(dev)
    out = torch.zeros(1, m, n, dtype=torch.bfloat16, device=dev)
    outs = (ctypes.c_void_p * 1)(out.data_ptr())
    devices = (ctypes.c_int * 1)(torch.cuda.current_device())
    args = lambda world, channel: (_ptr(x), x.stride(0), 1, _ptr(codes), _ptr(scales), 0, _ptr(inverse), outs, devices,
                                   world, 0, channel, 0, 1, m, n, k, None)
    assert lib.dg_enqueue_nvfp4_allgather_noalloc(*args(1, 64)) == 1      # channel past the 64 built-in blocks
    assert lib.dg_enqueue_nvfp4_allgather_noalloc(*args(1, -1)) == 1
    assert lib.dg_enqueue_nvfp4_allgather_noalloc(*args(9, 0)) == 1       # more ranks than the counters cover
    assert lib.dg_enqueue_nvfp4_allgather_noalloc(*args(1, 63)) == 0      # the last channel works
    torch.cuda.synchronize()
    assert lib.dg_take_status() == 0
    # signal-only slots are refused: nothing could collect their arrivals from the built-in counters
    for slot in (2, 3):
        assert lib.dg_enqueue_nvfp4_allgather_noalloc(_ptr(x), x.stride(0), 1, _ptr(codes), _ptr(scales), 0,
                                                      _ptr(inverse), outs, devices, 1, 0, 5, slot, 1, m, n, k, None) == 1
    # the rank's device must be the current one
    other = (ctypes.c_int * 1)(torch.cuda.current_device() + 1)
    assert lib.dg_enqueue_nvfp4_allgather_noalloc(_ptr(x), x.stride(0), 1, _ptr(codes), _ptr(scales), 0, _ptr(inverse),
                                                  outs, other, 1, 0, 5, 0, 1, m, n, k, None) == 1
    # a channel can be put back to zero in stream order, and works afterwards
    assert lib.dg_reset_noalloc_channel(5, None) == 0
    assert lib.dg_reset_noalloc_channel(64, None) == 1
    assert lib.dg_enqueue_nvfp4_allgather_noalloc(*args(1, 5)) == 0
    torch.cuda.synchronize()
    assert lib.dg_take_status() == 0
