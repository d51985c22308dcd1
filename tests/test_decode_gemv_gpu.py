"""GPU parity tests: the CUDA GEMVs against the CPU oracle (FP64 product of the stored values), bit-exact row
invariance, refusals, graph capture, both scale layouts: the cases of the reference's own test file
(decode-gemv/tests/test_decode_gemv.py) at its shapes and bounds, through the C ABI and through the torch ops, plus
what a column-sharded stack relies on (a slice of the rows gives the whole matrix's bits) and guard bands."""
import numpy as np
import pytest
import torch

from oracle import decode_gemv_oracle as oc
from oracle import workloads as wl
from tests import helpers as h

pytestmark = pytest.mark.gpu
dev = torch.device("cuda")


def nr():
    import crit_kernels_b200
    return crit_kernels_b200.get_kernel("crit-labs/decode-gemv", version=1)


def cuda(*ts):
    return tuple(t.to(dev) for t in ts)


def gemv_abi(fmt, x, tensors, dtype=torch.float32, blocked=False):
    out = torch.empty(x.shape[0], tensors[0].shape[0], dtype=dtype, device=dev)
    return h.run(fmt, x, tensors, out, blocked=blocked)


def check_rows(fmt, x, tensors, batch, **kw):
    """Every row count 1..16: each row of the batched call equals the same row alone (a clone at another address)."""
    for rows in range(1, x.shape[0] + 1):
        part = gemv_abi(fmt, x[:rows], tensors, **kw)
        assert torch.equal(part, batch[:rows]), (fmt, rows)
        alone = gemv_abi(fmt, x[rows - 1:rows].clone(), tensors, **kw)
        assert torch.equal(alone[0], batch[rows - 1]), (fmt, rows)


# ----- NVFP4 -----------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("shape", [(96, 256), (1000, 5120), (130, 2048)])
def test_nvfp4_multiplies_by_the_stored_values_and_keeps_rows(shape):
    n, k = shape
    host = wl.ref_nvfp4(n, k)
    t = cuda(*host)
    x = wl.activations(16, k).to(dev)
    batch = gemv_abi("nvfp4", x, t)
    assert oc.within_fp32_bound(batch, x, oc.nvfp4_values(*host))       # 2e-5 of sum |x||w|, as the reference
    check_rows("nvfp4", x, t, batch)
    assert torch.equal(gemv_abi("nvfp4", x, t), batch)                   # a repeat


def test_nvfp4_16_bit_outputs_and_fp16_activations():
    host = wl.ref_nvfp4(96, 256)
    t = cuda(*host)
    x = wl.activations(3, 256).to(dev)
    full = gemv_abi("nvfp4", x, t)
    assert torch.equal(gemv_abi("nvfp4", x, t, torch.bfloat16), full.to(torch.bfloat16))   # one rounding
    half = gemv_abi("nvfp4", x.half(), t, torch.float16)
    exact = oc.gemv_exact(x.half(), oc.nvfp4_values(*host))
    assert oc.max_rel_error(half, exact) < 1e-3


@pytest.mark.parametrize("shape", [(96, 256), (130, 2080), (1000, 5120)])
def test_nvfp4_blocked_scales_give_the_row_major_bits(shape):
    n, k = shape
    codes, scales, inverse = wl.ref_nvfp4(n, k)
    c, s, i = cuda(codes, scales, inverse)
    blocked = oc.to_blocked(scales).to(dev)
    x = wl.activations(16, k).to(dev)
    for rows in (1, 5, 16):
        want = gemv_abi("nvfp4", x[:rows], (c, s, i))
        found = gemv_abi("nvfp4", x[:rows], (c, blocked, i), blocked=True)
        assert torch.equal(found, want), (shape, rows)
    assert oc.within_fp32_bound(want, x, oc.nvfp4_values(codes, scales, inverse))


def test_nvfp4_direct_and_staged_scale_paths_agree():
    """K a multiple of 256 stages scale rows by bulk copy; a scale pointer off 16 bytes reads them directly."""
    n, k = 200, 1024
    codes, scales, inverse = wl.ref_nvfp4(n, k)
    c, s, i = cuda(codes, scales, inverse)
    x = wl.activations(7, k).to(dev)
    staged = gemv_abi("nvfp4", x, (c, s, i))
    shifted = torch.empty(n * (k // 16) + 2, dtype=torch.uint8, device=dev)[2:].view(n, k // 16)
    shifted.copy_(s)
    assert shifted.data_ptr() % 16 == 2
    assert torch.equal(gemv_abi("nvfp4", x, (c, shifted, i)), staged)


# ----- FP8 / MXFP8 -------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("mx", [False, True])
@pytest.mark.parametrize("shape", [(96, 256), (1024, 5120), (130, 2048)])
def test_fp8_multiplies_by_the_stored_values_and_keeps_rows(mx, shape):
    n, k = shape
    fmt = "mxfp8" if mx else "fp8"
    host = wl.ref_fp8(n, k, mx)
    t = cuda(*host)
    x = wl.activations(16, k).to(dev)
    values = oc.fp8_values(*host)
    out = gemv_abi(fmt, x, t)
    assert oc.within_fp32_bound(out, x, values)
    check_rows(fmt, x, t, out)
    small = (x[:3] / 64).half()      # FP16 out: keep the sums inside FP16's range
    half = gemv_abi(fmt, small, t, torch.float16)
    assert oc.max_rel_error(half, oc.gemv_exact(small, values)) < 2e-3


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8"])
def test_activations_outside_fp16_range_keep_the_bits(fmt):
    """At few activation rows the FP8 / NVFP4 kernels hold BF16 activations as FP16 wherever a 512-byte step of them
    converts exactly (up to 65504, eight significant bits down to 2^-17, FP16 subnormals below) and as BF16 elsewhere.
    Rows must not change with that choice: activations with tiny, subnormal and huge values in some steps (and all of
    one row) against the same rows in a 16-row call, whose kernel never converts them, and against the exact
    product."""
    n, k = 300, 4096
    host = wl.ref_nvfp4(n, k) if fmt == "nvfp4" else wl.ref_fp8(n, k, False)
    values = oc.nvfp4_values(*host) if fmt == "nvfp4" else oc.fp8_values(*host)
    t = cuda(*host)
    x = wl.activations(16, k).clone()
    x[0, 5] = 1e-30                       # far below FP16: the step stays BF16
    x[0, 1500] = 3e-6                     # between FP16 subnormals: stays BF16 too
    x[0, 1800] = 2.0 ** -22               # an FP16 subnormal, exactly: fits
    x[0, 2100] = 0.0                      # zero fits
    x[1, 3000] = 70000.0                  # above FP16's largest
    x[1, 3001] = -2.0 ** -14              # the smallest normal fits
    x[2] = x[2] * 2.0 ** -20              # a whole row of small values
    x[3, 4095] = 1e-40                    # a BF16 subnormal
    x = x.to(torch.bfloat16).to(dev)
    batch = gemv_abi(fmt, x, t)
    assert oc.max_rel_error(batch.cpu(), oc.gemv_exact(x.cpu(), values)) < 1e-4
    for rows in (1, 2, 3, 4):
        part = gemv_abi(fmt, x[:rows], t)
        assert torch.equal(part, batch[:rows]), (fmt, rows)
    for row in range(4):
        alone = gemv_abi(fmt, x[row:row + 1].clone(), t)
        assert torch.equal(alone[0], batch[row]), (fmt, row)
    assert h.cabi.load().dg_take_status() == 0


def test_mxfp8_direct_and_staged_scale_paths_agree():
    n, k = 100, 1024
    codes, mx = wl.ref_fp8(n, k, True)
    c, s = cuda(codes, mx)
    x = wl.activations(5, k).to(dev)
    staged = gemv_abi("mxfp8", x, (c, s))
    shifted = torch.empty(n * (k // 32) + 1, dtype=torch.uint8, device=dev)[1:].view(n, k // 32)
    shifted.copy_(s)
    assert torch.equal(gemv_abi("mxfp8", x, (c, shifted)), staged)
    # K not a multiple of 512 always reads directly
    codes2, mx2 = wl.ref_fp8(40, 1312, True)
    x2 = wl.activations(3, 1312).to(dev)
    out = gemv_abi("mxfp8", x2, cuda(codes2, mx2))
    assert oc.within_fp32_bound(out, x2, oc.fp8_values(codes2, mx2))


def test_e8m0_edge_exponents():
    """Exponent byte 0 is 2^-127 (an FP32 subnormal scale), 254 is 2^127, 255 gives NaN: decode_gemv.cu:275-278."""
    n, k = 16, 64
    codes = torch.full((n, k), 0x38, dtype=torch.uint8)          # E4M3 1.0
    mx = torch.full((n, k // 32), 127, dtype=torch.uint8)
    mx[1, 0] = 0
    mx[2, 1] = 254
    mx[3, 0] = 255
    x = torch.zeros(1, k, dtype=torch.bfloat16)
    x[0, 0] = 2.0 ** 100
    x[0, 32] = 2.0 ** -100
    out = gemv_abi("mxfp8", x.to(dev), cuda(codes, mx)).cpu()[0]
    assert out[0] == 2.0 ** 100 + 2.0 ** -100
    assert out[1] == np.float32(2.0 ** -27) + np.float32(2.0 ** -100)
    assert out[2] == np.float32(2.0 ** 100) + np.float32(2.0 ** 27)
    assert torch.isnan(out[3]) and not torch.isnan(out[4:]).any()


# ----- BF16 --------------------------------------------------------------------------------------------------------

def test_bf16_multiplies_and_keeps_rows():
    w = wl.ref_bf16(1000, 2048).to(dev)
    x = wl.activations(16, 2048).to(dev)
    exact = oc.gemv_exact(x, oc.bf16_values(w))
    out = gemv_abi("bf16", x, (w,))
    assert oc.max_rel_error(out, exact) < 1e-5
    check_rows("bf16", x, (w,), out)
    assert torch.equal(gemv_abi("bf16", x, (w,), torch.bfloat16), out.to(torch.bfloat16))


# ----- shapes at the edges ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("fmt,n,k", [("bf16", 1, 8), ("bf16", 5, 264), ("fp8", 1, 16), ("fp8", 7, 48), ("fp8", 23, 4112),
                                     ("mxfp8", 3, 32), ("mxfp8", 9, 4128), ("nvfp4", 1, 32), ("nvfp4", 13, 2080),
                                     ("nvfp4", 29, 8224), ("nvfp4", 2000, 64), ("fp8", 1500, 528), ("bf16", 1100, 40)])
@pytest.mark.parametrize("m", [1, 3, 16])
def test_small_and_ragged_shapes(fmt, n, k, m):
    host = {"nvfp4": lambda: wl.ref_nvfp4(n, k), "fp8": lambda: wl.ref_fp8(n, k, False),
            "mxfp8": lambda: wl.ref_fp8(n, k, True), "bf16": lambda: (wl.ref_bf16(n, k),)}[fmt]()
    x = wl.activations(m, k).to(dev)
    # guard bands: the output lives inside a larger buffer that must stay untouched around it
    ldo = n + 24
    buf = torch.full((m + 2, ldo), -7.0, device=dev)
    out = buf[1:m + 1, 8:8 + n]
    h.run(fmt, x, cuda(*host), out)
    assert oc.within_fp32_bound(out, x, oc.values_of(fmt, host))
    mask = torch.ones_like(buf, dtype=torch.bool)
    mask[1:m + 1, 8:8 + n] = False
    assert bool((buf[mask] == -7.0).all())


def test_strided_activations():
    n, k = 300, 1024
    host = wl.ref_fp8(n, k, False)
    wide = torch.zeros(6, k + 64, dtype=torch.bfloat16, device=dev)
    x = wl.activations(6, k).to(dev)
    wide[:, 32:32 + k] = x
    view = wide[:, 32:32 + k]           # row stride K + 64, base offset 64 bytes
    assert torch.equal(gemv_abi("fp8", view, cuda(*host)), gemv_abi("fp8", x, cuda(*host)))


# ----- what a column-sharded stack relies on -----------------------------------------------------------------------

@pytest.mark.parametrize("fmt,n,k", [("nvfp4", 1024, 2048), ("fp8", 1024, 2048), ("mxfp8", 1024, 2048),
                                     ("bf16", 1024, 1024)])
def test_a_slice_of_the_rows_gives_the_whole_matrix_bits(fmt, n, k):
    host = {"nvfp4": lambda: wl.cfg_nvfp4(n, k), "fp8": lambda: wl.cfg_fp8(n, k),
            "mxfp8": lambda: wl.cfg_mxfp8(n, k), "bf16": lambda: (wl.cfg_bf16(n, k),)}[fmt]()
    t = cuda(*host)
    x = wl.activations(8, k).to(dev)
    whole = gemv_abi(fmt, x, t, torch.bfloat16)
    for parts in (2, 4, 8):
        rows = n // parts
        pieces = [gemv_abi(fmt, x, tuple(a[r * rows:(r + 1) * rows].contiguous() for a in t), torch.bfloat16)
                  for r in range(parts)]
        assert torch.equal(torch.cat(pieces, dim=1), whole), (fmt, parts)


# ----- the torch op surface ------------------------------------------------------------------------------------------

def test_ops_give_the_abi_bits_and_return_out():
    k = nr()
    c, s, i = cuda(*wl.ref_nvfp4(130, 2048))
    x = wl.activations(9, 2048).to(dev)
    out = torch.empty(9, 130, device=dev)
    assert k.gemv(x, c, s.view(torch.float8_e4m3fn), i, out) is out
    assert torch.equal(out, gemv_abi("nvfp4", x, (c, s, i)))
    fc, fs = cuda(*wl.ref_fp8(130, 2048, False))
    out8 = torch.empty(9, 130, device=dev)
    k.gemv_fp8(x, fc.view(torch.float8_e4m3fn), fs, out8)
    assert torch.equal(out8, gemv_abi("fp8", x, (fc, fs)))
    w = wl.ref_bf16(130, 2048).to(dev)
    out16 = torch.empty(9, 130, device=dev, dtype=torch.bfloat16)
    k.gemv_bf16(x, w, out16)
    assert torch.equal(out16, gemv_abi("bf16", x, (w,), torch.bfloat16))
    assert k.hardware_decode() is True and k.hardware_decode(dev) is True


def test_ops_refuse_what_they_cannot_read():
    k = nr()
    c, s, i = cuda(*wl.ref_nvfp4(96, 256))
    x = wl.activations(9, 256).to(dev)
    out = lambda m: torch.empty(m, 96, device=dev)
    with pytest.raises(RuntimeError):
        k.gemv(wl.activations(17, 256).to(dev), c, s, i, out(17))                 # 17 rows
    with pytest.raises(RuntimeError):
        k.gemv(wl.activations(2, 260).to(dev)[:, 4:], c, s, i, out(2))           # rows off 16-byte boundaries
    with pytest.raises(RuntimeError):
        k.gemv(x[:2].float(), c, s, i, out(2))                                    # FP32 activations
    with pytest.raises(RuntimeError):
        k.gemv(x[:2], c, s, i.cpu(), out(2))                                      # another device
    odd = torch.empty(96 * 16 + 1, dtype=torch.uint8, device=dev)[1:].view(96, 16)
    odd.copy_(s)
    with pytest.raises(RuntimeError):
        k.gemv(x[:2], c, odd, i, out(2))                                          # scales off 2 bytes
    blocked = oc.to_blocked(s.cpu()).to(dev)
    with pytest.raises(RuntimeError):
        k.gemv(x[:2], c, blocked[:-4], i, out(2), blocked=True)                   # truncated tiled scales
    with pytest.raises(RuntimeError):
        k.gemv(x[:2], c, s, i, torch.empty(2, 96, device=dev, dtype=torch.float16))   # out neither FP32 nor x's
    fc, fs = cuda(*wl.ref_fp8(96, 256, False))
    with pytest.raises(RuntimeError):
        k.gemv_fp8(x[:2], fc, fs[:10], out(2))                                    # a scale per row
    mc, ms = cuda(*wl.ref_fp8(96, 256, True))
    with pytest.raises(RuntimeError):
        k.gemv_fp8(x[:2], mc, ms[:, :4], out(2))                                  # an exponent per 32 inputs
    with pytest.raises(RuntimeError):
        k.gemv_fp8(x[:2].float(), fc, fs, out(2))
    with pytest.raises(RuntimeError):
        k.gemv_fp8(x[:2], fc, fs.cpu(), out(2))
    with pytest.raises(RuntimeError):
        k.gemv_bf16(x[:2].half(), wl.ref_bf16(96, 256).to(dev), out(2))          # BF16 activations only


def test_the_gemvs_capture_in_a_cuda_graph():
    k = nr()
    c, s, i = cuda(*wl.ref_nvfp4(1000, 2048))
    fc, fs = cuda(*wl.ref_fp8(1000, 2048, True))
    w = wl.ref_bf16(1000, 2048, seed=1).to(dev)
    x = wl.activations(4, 2048).to(dev)
    outs = [torch.empty(4, 1000, device=dev) for _ in range(3)]
    k.gemv(x, c, s, i, outs[0])
    k.gemv_fp8(x, fc, fs, outs[1])
    k.gemv_bf16(x, w, outs[2])
    eager = [o.clone() for o in outs]
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        k.gemv(x, c, s, i, outs[0])
        k.gemv_fp8(x, fc, fs, outs[1])
        k.gemv_bf16(x, w, outs[2])
    for o in outs:
        o.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for o, e in zip(outs, eager):
        assert torch.equal(o, e)


def test_no_bounded_wait_ran_out():
    """After everything above, the kernels' error word is clean."""
    from crit_kernels_b200 import cabi
    assert cabi.load().dg_take_status() == 0


def test_one_rank_allgather_is_the_plain_gemv():
    """The all-gather entry point with a single rank: results land in slot 0 of the gathered buffer, bit-identical
    to the plain GEMV, and the arrival counters are back at zero after every call."""
    import ctypes
    from crit_kernels_b200 import cabi
    n, k, m = 520, 2048, 5
    c, s, i = cuda(*wl.cfg_nvfp4(n, k))
    x = wl.activations(m, k).to(dev)
    want = gemv_abi("nvfp4", x, (c, s, i), torch.bfloat16)
    full = torch.zeros(1, m, n, dtype=torch.bfloat16, device=dev)
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    outs = (ctypes.c_void_p * 1)(full.data_ptr())
    flag_ptrs = (ctypes.c_void_p * 1)(flags.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(4):
        full.zero_()
        code = cabi.load().dg_enqueue_nvfp4_allgather(ptr(x), x.stride(0), 1, ptr(c), ptr(s), 0, ptr(i), outs, flag_ptrs,
                                                      1, 0, call & 1, 1, m, n, k, stream)
        assert code == 0
        torch.cuda.synchronize()
        assert torch.equal(full[0], want) and int(flags.abs().sum()) == 0
    assert cabi.load().dg_take_status() == 0


@pytest.mark.parametrize("m", [4, 9])   # kernels with producer warps; kernels whose consumers issue the copies
def test_static_weight_prefetch_gives_the_same_bits(m):
    """dg_set_static_weights(1) lets a GEMV stream weights before the previous kernel of the stream has finished; the
    results of back-to-back GEMVs whose activations are the previous GEMV's outputs stay bit-identical."""
    from crit_kernels_b200 import cabi
    k = nr()
    n = 2048
    c1, s1, i1 = cuda(*wl.cfg_nvfp4(n, n, seed=1))
    c2, s2, i2 = cuda(*wl.cfg_nvfp4(n, n, seed=2))
    fc, fs = cuda(*wl.cfg_fp8(n, n, seed=3))
    x = wl.activations(m, n).to(dev)

    def chain():
        a = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        b = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        for _ in range(3):                      # each GEMV reads what the one before it wrote
            k.gemv(x, c1, s1, i1, a)
            k.gemv(a, c2, s2, i2, b)
            k.gemv_fp8(b, fc, fs, c)
        torch.cuda.synchronize()
        return a, b, c

    want = chain()
    previous = cabi.load().dg_set_static_weights(1)
    try:
        found = chain()
    finally:
        cabi.load().dg_set_static_weights(previous)
    for f, w in zip(found, want):
        assert torch.equal(f, w)
    assert cabi.load().dg_take_status() == 0


def test_a_wait_that_runs_out_reports_and_leaves_the_device_usable():
    """No arrival ever comes for this counter: with the wait limit set to a millisecond the waiting kernel gives up,
    sets status bit 2 and returns; after the counters are re-zeroed a normal gathered call is clean."""
    import ctypes
    from crit_kernels_b200 import cabi
    lib = cabi.load()
    dev = torch.device("cuda")
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    previous = lib.dg_set_wait_limit_ns(1_000_000)
    try:
        assert lib.dg_enqueue_gather_wait(ctypes.c_void_p(flags.data_ptr()), 0, 1, None) == 0
        assert lib.dg_take_status() == 4                       # waited about 1 ms, gave up, said so
    finally:
        lib.dg_set_wait_limit_ns(previous)
    assert lib.dg_reset_counters(ctypes.c_void_p(flags.data_ptr()), None) == 0
    n, k, m = 300, 1024, 3
    codes, scales, inverse = (t.to(dev) for t in wl.cfg_nvfp4(n, k, seed=77))
    x = wl.activations(m, k, seed=78).to(dev)
    want = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    h.run("nvfp4", x, (codes, scales, inverse), want)
    got = torch.zeros(1, m, n, dtype=torch.bfloat16, device=dev)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    assert lib.dg_enqueue_nvfp4_allgather(ptr(x), x.stride(0), 1, ptr(codes), ptr(scales), 0, ptr(inverse),
                                          (ctypes.c_void_p * 1)(got.data_ptr()),
                                          (ctypes.c_void_p * 1)(flags.data_ptr()), 1, 0, 0, 1, m, n, k, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(got[0].view(torch.int16), want.view(torch.int16))
    assert lib.dg_take_status() == 0
