"""GPU parity tests of the NVFP4 dequantizers (decode, decode_fp8): bit-exact against the CPU oracle and against the
golden vectors made from the reference test's own expectation (decode-gemv/tests/test_decode_gemv.py:131-140), through
the C ABI and through the package functions; ragged sizes, refusals, graph capture, and at full size the consistency
of dequantize-then-GEMV with the NVFP4 GEMV."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import decode_gemv_oracle as oc
from oracle import workloads as wl

pytestmark = pytest.mark.gpu
dev = torch.device("cuda")
KIND = {torch.bfloat16: 1, torch.float16: 2, torch.float8_e4m3fn: 3}


def nr():
    import crit_kernels_b200
    return crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)


def abi_dequantize(codes, scales, factor, dtype):
    from crit_kernels_b200 import cabi
    n, k = codes.shape[0], codes.shape[1] * 2
    out = torch.empty(n, k, dtype=dtype, device=dev)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = cabi.load().dg_enqueue_dequantize(ptr(codes), ptr(scales), ptr(factor), ptr(out), KIND[dtype], n, k, stream)
    assert code == 0, f"cudaError {code}"
    return out


def bits(t):
    return t.view(torch.uint8 if t.element_size() == 1 else torch.int16).cpu()


@pytest.mark.parametrize("tag", ["a", "b"])
def test_golden_vectors_of_the_reference_test(golden, tag):
    c, s, i = (torch.from_numpy(golden[f"nvfp4_{tag}_{p}"]).to(dev) for p in ("codes", "scales", "inverse"))
    assert np.array_equal(bits(abi_dequantize(c, s, i, torch.bfloat16)).numpy(), golden[f"nvfp4_{tag}_decode_bf16"])
    assert np.array_equal(bits(abi_dequantize(c, s, i, torch.float16)).numpy(), golden[f"nvfp4_{tag}_decode_f16"])
    assert np.array_equal(bits(abi_dequantize(c, s, i * 64, torch.float8_e4m3fn)).numpy(),
                          golden[f"nvfp4_{tag}_decode_fp8"])


def test_the_decoders_round_one_fp32_product_once():
    """The reference's own case (tests/test_decode_gemv.py:131-140), through the package functions."""
    k = nr()
    c, s, i = wl.ref_nvfp4(96, 256)
    unit = torch.from_numpy(oc.nvfp4_values(c, s, torch.ones_like(i))).float()        # e2m1 * scale, exact in FP32
    product = (unit * i[:, None]).to(dev)
    cd, sd, idev = c.to(dev), s.to(dev), i.to(dev)
    for dtype in (torch.bfloat16, torch.float16):
        out = torch.empty(96, 256, dtype=dtype, device=dev)
        assert k.decode(cd, sd, idev, out) is out
        assert torch.equal(out, product.to(dtype)), dtype
    factor = idev * 64
    out = torch.empty(96, 256, dtype=torch.float8_e4m3fn, device=dev)
    want = (unit.to(dev) * factor[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(k.decode_fp8(cd, sd, factor, out).view(torch.uint8), want.view(torch.uint8))


@pytest.mark.parametrize("shape", [(1, 16), (3, 48), (130, 544), (257, 2064), (40, 16400), (70000, 32)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float8_e4m3fn])
def test_ragged_sizes_match_the_oracle_bit_for_bit(shape, dtype):
    n, k = shape
    c, s, i = wl.cfg_nvfp4(n, k, seed=n + k)
    i = i * (48.0 if dtype == torch.float8_e4m3fn else 1.0)      # some FP8 values saturate
    found = abi_dequantize(c.to(dev), s.to(dev), i.to(dev), dtype)
    assert torch.equal(bits(found), bits(oc.dequantize(c, s, i, dtype)))
    torch.cuda.synchronize()


def test_every_code_and_every_scale_byte():
    """All 256 code bytes against all 256 E4M3 scale bytes (NaN scales included): FP32 bit patterns agree with the
    oracle after the rounding to each output type."""
    codes = torch.arange(256, dtype=torch.uint8).repeat_interleave(8).reshape(256, 8)   # a 16-value block of one byte
    codes = codes.repeat(256, 1)                                                           # row = (scale, code byte)
    scales = torch.arange(256, dtype=torch.uint8).repeat_interleave(256).reshape(-1, 1)
    factor = torch.full((65536,), 0.75, dtype=torch.float32)
    for dtype in (torch.bfloat16, torch.float16, torch.float8_e4m3fn):
        found = abi_dequantize(codes.to(dev), scales.to(dev), factor.to(dev), dtype).cpu()
        want = oc.dequantize(codes, scales, factor, dtype)
        same = (bits(found) == bits(want)) | (found.float().isnan() & want.float().isnan())
        assert bool(same.all()), dtype


def test_refusals():
    from crit_kernels_b200 import cabi
    k = nr()
    c, s, i = (t.to(dev) for t in wl.cfg_nvfp4(8, 64))
    out = torch.empty(8, 64, dtype=torch.bfloat16, device=dev)
    with pytest.raises(RuntimeError):
        k.decode(c, s, i, torch.empty(8, 64, dtype=torch.float32, device=dev))          # 32-bit output
    with pytest.raises(RuntimeError):
        k.decode_fp8(c, s, i, out)                                                        # not FP8
    with pytest.raises(RuntimeError):
        k.decode(c, s, i, torch.empty(8, 48, dtype=torch.bfloat16, device=dev))          # K does not match the codes
    with pytest.raises(RuntimeError):
        k.decode(c, s, i[:7], out)                                                        # one factor per row
    with pytest.raises(RuntimeError):
        k.decode(c, s[:, :3], i, out)                                                     # scales [N][K / 16]
    with pytest.raises(RuntimeError):
        k.decode(c, s, i, torch.empty(8, 128, dtype=torch.bfloat16, device=dev)[:, ::2])  # not contiguous
    with pytest.raises(RuntimeError):
        k.decode(c.cpu(), s, i, out)                                                      # host tensor
    lib, p0 = cabi.load(), ctypes.c_void_p(out.data_ptr())
    assert lib.dg_enqueue_dequantize(p0, p0, p0, p0, 1, 8, 24, None) != 0                 # K not a multiple of 16
    assert lib.dg_enqueue_dequantize(p0, p0, p0, p0, 0, 8, 64, None) != 0                 # unknown output type
    assert lib.dg_enqueue_dequantize(p0, p0, p0, p0, 1, 0, 64, None) != 0                 # no rows
    assert lib.dg_enqueue_dequantize(None, p0, p0, p0, 1, 8, 64, None) != 0               # null codes
    torch.cuda.synchronize()


def test_captures_in_a_cuda_graph():
    k = nr()
    c, s, i = (t.to(dev) for t in wl.cfg_nvfp4(1000, 2048))
    out = torch.empty(1000, 2048, dtype=torch.bfloat16, device=dev)
    eager = k.decode(c, s, i, out).clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        k.decode(c, s, i, out)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        k.decode(c, s, i, out)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


def test_full_size_dequantize_then_gemv_agrees_with_the_nvfp4_gemv():
    """28672 x 8192 (235 M values): sampled rows bit-equal to the oracle, and gemv_bf16 over the dequantized matrix
    within BF16 rounding of the weights of the NVFP4 GEMV (the reference's dequantize-then-matmul cross-check)."""
    k = nr()
    n, kk = 28672, 8192
    c, s, i = wl.cfg_nvfp4(n, kk, seed=11)
    cd, sd, idev = c.to(dev), s.to(dev), i.to(dev)
    w = torch.empty(n, kk, dtype=torch.bfloat16, device=dev)
    k.decode(cd, sd, idev, w)
    rows = torch.tensor([0, 1, 127, 128, 4097, 14335, 28670, 28671])
    want = oc.dequantize(c[rows], s[rows], i[rows], torch.bfloat16)
    assert torch.equal(w[rows.to(dev)].cpu(), want)
    x = wl.activations(4, kk).to(dev)
    direct = torch.empty(4, n, dtype=torch.float32, device=dev)
    via = torch.empty(4, n, dtype=torch.float32, device=dev)
    k.gemv(x, cd, sd, idev, direct)
    k.gemv_bf16(x, w, via)
    assert float((direct - via).abs().max() / direct.abs().max()) < 1e-2      # BF16 rounding of every weight
    w8 = torch.empty(n, kk, dtype=torch.float8_e4m3fn, device=dev)
    k.decode_fp8(cd, sd, idev * 32, w8)
    want8 = oc.dequantize(c[rows], s[rows], i[rows] * 32, torch.float8_e4m3fn)
    assert torch.equal(w8[rows.to(dev)].view(torch.uint8).cpu(), want8.view(torch.uint8))
