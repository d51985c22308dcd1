"""The activation quantizers (dg_enqueue_quantize_fp8_rows, dg_enqueue_quantize_nvfp4) on a B200, bit for bit against
the CPU oracle, against the reference tests' torch expressions evaluated on the device
(mma-rows/tests/test_mma_rows.py:80-104, the reference's own check at :153-174) and, where oracle/_ref holds it,
against the reference's unmodified kernels on the same inputs."""
import ctypes

import numpy as np
import pytest
import torch

import crit_kernels_b200
from crit_kernels_b200 import cabi
from oracle import build_ref
from oracle import decode_gemv_oracle as oc
from oracle import quantize_oracle as qo

pytestmark = pytest.mark.gpu
INPUT_SCALE = 300.0
BOUNDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
TIES = torch.tensor([0.75, 1.75, 3.5])


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def torch_fp8_rows(x):
    """Per-row FP8 as a framework writes it on the device."""
    x = x.float()
    scale = (x.abs().amax(dim=-1) / 448.0).clamp(min=1e-12)
    return (x / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8), scale


def torch_nvfp4(x, input_scale):
    x = x.float()
    t, k = x.shape
    blocks = x.view(t, k // 16, 16)
    scale = (blocks.abs().amax(dim=-1) / 6.0 * input_scale).clamp(max=448.0).to(torch.float8_e4m3fn)
    decoded = scale.float() / input_scale
    scaled = torch.where(decoded[..., None] > 0, blocks / decoded[..., None].clamp(min=1e-30), torch.zeros_like(blocks))
    magnitude = scaled.abs().clamp(max=6.0)
    code = torch.bucketize(magnitude, BOUNDS.to(x.device), right=False)
    code = code + torch.isin(magnitude, TIES.to(x.device)).to(code.dtype)
    code = (code | ((scaled < 0).to(code.dtype) << 3)).to(torch.uint8).view(t, k)
    return code[:, 0::2] | (code[:, 1::2] << 4), scale.view(torch.uint8)


def inputs(m, k, seed, spread=False):
    """[m][k] BF16 as a view of rows that are a multiple of 8 values apart (what the ops require of any K)."""
    g = torch.Generator().manual_seed(seed)
    wide = (k + 7) // 8 * 8
    x = torch.randn(m, wide, generator=g) * 3
    if spread:
        x = x * torch.exp2(torch.randint(-24, 8, (m, (wide + 15) // 16), generator=g).float()
                           ).repeat_interleave(16, dim=1)[:, :wide]
    return x.to(torch.bfloat16)


def on_device(wide, k):
    """The first k columns of the wide batch on the GPU, rows still a multiple of 8 values apart."""
    return wide.to(torch.device("cuda"))[:, :k]


@pytest.mark.parametrize("m,k,spread", [(37, 2048, False), (1, 8192, False), (5, 1001, False), (3, 20000, False),
                                        (16, 28672, False), (9, 512, True), (2, 7, False), (130, 640, True),
                                        (2, 120000, False)])
def test_fp8_rows_match_the_oracle_and_the_torch_expression(m, k, spread):
    dev = torch.device("cuda")
    k_mod = crit_kernels_b200.get_kernel()
    wide = inputs(m, k, 100 + m + k, spread)
    if m > 3:
        wide[3, : min(100, k)] = 0
    x, xd = wide[:, :k], on_device(wide, k)
    q = torch.full((m, k), 0x55, dtype=torch.uint8, device=dev)
    scale = torch.empty(m, dtype=torch.float32, device=dev)
    k_mod.quantize_fp8_rows(xd, q, scale)
    torch.cuda.synchronize()
    want_q, want_scale = qo.fp8_rows(x)
    assert np.array_equal(scale.cpu().numpy().view(np.uint32), want_scale.view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), want_q)
    tq, ts = torch_fp8_rows(xd)
    assert torch.equal(scale, ts) and torch.equal(q, tq)


def test_fp8_rows_take_strided_and_unaligned_buffers():
    dev = torch.device("cuda")
    lib = cabi.load()
    m, k = 6, 1000
    x = inputs(m, k + 24, 7).to(dev)
    want_q, want_scale = qo.fp8_rows(x[:, 8:8 + k].cpu())
    for q_pad, q_off in ((0, 0), (24, 0), (13, 3)):                  # vector stores, padded rows, byte stores
        q = torch.full((m, k + q_pad + q_off), 0x55, dtype=torch.uint8, device=dev)
        scale = torch.empty(m, dtype=torch.float32, device=dev)
        xv, qv = x[:, 8:8 + k], q[:, q_off:q_off + k]
        assert lib.dg_enqueue_quantize_fp8_rows(_ptr(xv), xv.stride(0), m, k, _ptr(qv), qv.stride(0), _ptr(scale),
                                                None) == 0
        torch.cuda.synchronize()
        assert np.array_equal(qv.cpu().numpy(), want_q) and np.array_equal(scale.cpu().numpy(), want_scale)
        rest = torch.ones_like(q, dtype=torch.bool)
        rest[:, q_off:q_off + k] = False
        assert bool((q[rest] == 0x55).all())                           # nothing written beside the rows
    # a row with a NaN gets a NaN scale, as torch's amax gives it
    y = inputs(2, 64, 9)
    y[1, 5] = float("nan")
    q = torch.empty(2, 64, dtype=torch.uint8, device=dev)
    scale = torch.empty(2, dtype=torch.float32, device=dev)
    crit_kernels_b200.get_kernel().quantize_fp8_rows(y.to(dev), q, scale)
    assert bool(torch.isnan(scale[1])) and not bool(torch.isnan(scale[0]))


@pytest.mark.parametrize("m,k,spread", [(37, 2048, False), (1, 8192, False), (5, 1008, False), (16, 28672, False),
                                        (9, 512, True), (130, 656, True), (200, 16, False), (1, 48, True)])
def test_nvfp4_matches_the_oracle_and_the_torch_expression(m, k, spread):
    dev = torch.device("cuda")
    k_mod = crit_kernels_b200.get_kernel()
    x = inputs(m, k, 300 + m + k, spread)
    if m > 3:
        x[3, : min(100, k)] = 0                                       # blocks of zeros: scale 0, codes 0
    if m > 8 and k >= 16:
        x[8, :16] = (torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.25, -0.75, -1.75, -3.5, 0.0, 1.0,
                                   -6.0]) * (6.0 / INPUT_SCALE)).to(torch.bfloat16)
    xd = x.to(dev)                                                    # K is a multiple of 16 here: rows stay aligned
    codes = torch.full((m, k // 2), 0x55, dtype=torch.uint8, device=dev)
    scales = torch.full((oc.blocked_numel(m, k),), 0x55, dtype=torch.uint8, device=dev)   # the padding is written too
    k_mod.quantize_nvfp4(xd, INPUT_SCALE, codes, scales)
    torch.cuda.synchronize()
    want_codes, want_blocked = qo.nvfp4_blocked(x, INPUT_SCALE)
    assert np.array_equal(codes.cpu().numpy(), want_codes)
    assert np.array_equal(scales.cpu().numpy(), want_blocked)
    tc, ts = torch_nvfp4(xd, INPUT_SCALE)
    assert torch.equal(codes, tc)
    assert torch.equal(scales.cpu(), oc.to_blocked(ts.cpu()))


def test_the_quantizers_give_the_bits_of_the_reference_kernels():
    ref = build_ref.load_quantizers()
    if ref is None:
        pytest.skip("oracle/_ref/libmma_rows_ref.so was not built (needs the reference checkout at build time)")
    dev = torch.device("cuda")
    lib = cabi.load()
    for m, k, spread in ((37, 2048, False), (5, 20000, False), (16, 8192, True), (3, 1001, False), (300, 1056, True)):
        x = on_device(inputs(m, k, 500 + m + k, spread), k)
        q1, q2 = (torch.zeros(m, k, dtype=torch.uint8, device=dev) for _ in range(2))
        s1, s2 = (torch.zeros(m, dtype=torch.float32, device=dev) for _ in range(2))
        assert lib.dg_enqueue_quantize_fp8_rows(_ptr(x), x.stride(0), m, k, _ptr(q1), k, _ptr(s1), None) == 0
        assert ref.ref_quantize_fp8_rows(_ptr(x), x.stride(0), m, k, _ptr(q2), k, _ptr(s2), None) == 0
        torch.cuda.synchronize()
        assert torch.equal(q1, q2) and torch.equal(s1.view(torch.int32), s2.view(torch.int32)), (m, k)
        if k % 16:
            continue
        c1, c2 = (torch.zeros(m, k // 2, dtype=torch.uint8, device=dev) for _ in range(2))
        b1, b2 = (torch.full((oc.blocked_numel(m, k),), 0x55, dtype=torch.uint8, device=dev) for _ in range(2))
        g = ctypes.c_float(INPUT_SCALE)
        r = ctypes.c_float(np.float32(1.0) / np.float32(INPUT_SCALE))
        assert lib.dg_enqueue_quantize_nvfp4(_ptr(x), x.stride(0), m, k, g, r, _ptr(c1), _ptr(b1), None) == 0
        assert ref.ref_quantize_nvfp4(_ptr(x), x.stride(0), m, k, g, r, _ptr(c2), _ptr(b2), None) == 0
        torch.cuda.synchronize()
        assert torch.equal(c1, c2) and torch.equal(b1, b2), (m, k)


def test_the_quantizers_refuse_what_they_cannot_read_and_capture_in_a_graph():
    dev = torch.device("cuda")
    k_mod = crit_kernels_b200.get_kernel()
    x = inputs(4, 256, 1).to(dev)
    q = torch.empty(4, 256, dtype=torch.uint8, device=dev)
    scale = torch.empty(4, dtype=torch.float32, device=dev)
    codes = torch.empty(4, 128, dtype=torch.uint8, device=dev)
    blocked = torch.empty(oc.blocked_numel(4, 256), dtype=torch.uint8, device=dev)
    with pytest.raises(RuntimeError):
        k_mod.quantize_fp8_rows(x.float(), q, scale)                   # FP32 activations
    with pytest.raises(RuntimeError):
        k_mod.quantize_fp8_rows(x, q[:, :100], scale)                  # wrong width
    with pytest.raises(RuntimeError):
        k_mod.quantize_fp8_rows(x, q, scale[:3])                       # wrong number of scales
    with pytest.raises(RuntimeError):
        k_mod.quantize_nvfp4(x[:, :40], INPUT_SCALE, codes[:, :20].contiguous(), blocked)    # K not a multiple of 16
    with pytest.raises(RuntimeError):
        k_mod.quantize_nvfp4(x, -1.0, codes, blocked)
    with pytest.raises(RuntimeError):
        k_mod.quantize_nvfp4(x, INPUT_SCALE, codes, blocked[:-4])      # truncated tiled scales
    with pytest.raises(RuntimeError):
        k_mod.quantize_nvfp4(x, INPUT_SCALE, codes.cpu(), blocked)
    k_mod.quantize_fp8_rows(x, q, scale)
    k_mod.quantize_nvfp4(x, INPUT_SCALE, codes, blocked)
    torch.cuda.synchronize()
    want = (q.clone(), scale.clone(), codes.clone(), blocked.clone())
    for t in (q, scale, codes, blocked):
        t.zero_()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        k_mod.quantize_fp8_rows(x, q, scale)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        k_mod.quantize_fp8_rows(x, q, scale)
        k_mod.quantize_nvfp4(x, INPUT_SCALE, codes, blocked)
    for t in (q, scale, codes, blocked):
        t.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for got, w in zip((q, scale, codes, blocked), want):
        assert torch.equal(got, w)
