"""Speed beside the unmodified reference kernel (oracle/_ref, built from the reference checkout for sm_100a): both
kernels on the same inputs, timed the same way (CUDA events around replays of a CUDA graph of 20 calls that rotate
over weight copies larger than the L2). Prints the table; asserts only that the B200 kernels are not slower than the
reference's by more than a margin, so that a regression shows up as a failure. Skipped when the reference library was
never built."""
import ctypes

import pytest
import torch

from oracle import build_ref
from oracle import workloads as wl
from tests import helpers as h

pytestmark = pytest.mark.gpu
dev = torch.device("cuda")

CASES = [("fp8", 1, 28672, 8192), ("fp8", 16, 28672, 8192), ("mxfp8", 1, 13824, 5120), ("bf16", 1, 16384, 8192),
         ("nvfp4", 1, 28672, 8192), ("nvfp4", 8, 8192, 28672), ("nvfp4", 1, 4096, 4096)]


def weights(fmt, n, k, copies):
    g = torch.Generator(device=dev).manual_seed(7)
    out = []
    for _ in range(copies):
        if fmt == "nvfp4":
            c = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=dev, generator=g)
            s = torch.exp2(torch.rand(n, k // 16, device=dev, generator=g) * 6 - 4).to(torch.float8_e4m3fn)
            out.append((c, s.view(torch.uint8), torch.ones(n, device=dev)))
        elif fmt == "fp8":
            c = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.float8_e4m3fn).view(torch.uint8)
            out.append((c, (torch.rand(n, device=dev, generator=g) * 1.5 + 0.5) / 64))
        elif fmt == "mxfp8":
            c = (torch.randn(n, k, device=dev, generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
            out.append((c.view(torch.uint8), torch.randint(110, 125, (n, k // 32), dtype=torch.uint8, device=dev,
                                                           generator=g)))
        else:
            out.append(((torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16),))
    return out


def reference_call(lib, fmt, x, t, out):
    p = lambda a: ctypes.c_void_p(a.data_ptr()) if a is not None else None
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    m, k = x.shape
    n = t[0].shape[0]
    if fmt == "nvfp4":
        return lib.ref_enqueue_nvfp4(p(x), x.stride(0), 1, p(t[0]), p(t[1]), 0, p(t[2]), p(out), out.stride(0), 1, m, n,
                                     k, stream)
    if fmt == "bf16":
        return lib.ref_enqueue_bf16(p(x), x.stride(0), p(t[0]), p(out), out.stride(0), 1, m, n, k, stream)
    mx = fmt == "mxfp8"
    return lib.ref_enqueue_fp8(p(x), x.stride(0), 1, p(t[0]), None if mx else p(t[1]), p(t[1]) if mx else None, p(out),
                               out.stride(0), 1, m, n, k, stream)


def graph_us(call, reps=5):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(3):
            call(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(20):
            call(i)
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (20 * reps) * 1e3


def test_not_slower_than_the_reference_kernel(capsys):
    lib = build_ref.load()
    if lib is None:
        pytest.skip("oracle/_ref/libdecode_gemv_ref.so was not built")
    rows = []
    for fmt, m, n, k in CASES:
        nbytes = wl.weight_bytes(fmt, n, k)
        copies = max(2, min(12, int(1.2e9 // nbytes)))
        ws = weights(fmt, n, k, copies)
        x = wl.activations(m, k).to(dev)
        ours_out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        ref_out = torch.empty_like(ours_out)
        ours = graph_us(lambda i: h.run(fmt, x, ws[i % copies], ours_out))
        theirs = graph_us(lambda i: reference_call(lib, fmt, x, ws[i % copies], ref_out))
        rows.append((fmt, m, n, k, ours, theirs, nbytes / ours / 1e3))
        del ws
        torch.cuda.empty_cache()
    with capsys.disabled():
        print("\nformat M N K: ours us (GB/s) | reference us | speed-up")
        for fmt, m, n, k, ours, theirs, gbs in rows:
            print(f"{fmt:6s} {m:2d} {n:6d} {k:6d}: {ours:8.2f} ({gbs:7.1f}) | {theirs:8.2f} | {theirs / ours:5.2f}x")
    for fmt, m, n, k, ours, theirs, _ in rows:
        assert ours <= theirs * 1.15, (fmt, m, n, k, ours, theirs)
