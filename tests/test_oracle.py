"""The CPU oracle against the reference's own test-side functions (golden vectors made from the reference test source
by tests/golden/make_golden.py) and against torch's FP8 dtypes."""
import numpy as np
import pytest
import torch

from oracle import decode_gemv_oracle as oc
from oracle import workloads as wl


def test_e2m1_table_is_the_references(golden):
    assert np.array_equal(oc.E2M1_TABLE, golden["e2m1_table"])
    assert np.array_equal(np.signbit(oc.E2M1_TABLE), np.signbit(golden["e2m1_table"]))


def test_e4m3_decode_matches_every_byte(golden):
    mine = oc.e4m3_to_float(np.arange(256, dtype=np.uint8))
    want = golden["e4m3_all"]
    assert np.array_equal(np.isnan(mine), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(mine[ok], want[ok])
    # and torch's cast today agrees with the stored table
    now = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).double().numpy()
    assert np.array_equal(now[ok], want[ok])


def test_e8m0_decode():
    e = np.arange(256, dtype=np.uint8)
    v = oc.e8m0_to_float(e)
    assert v[0] == 2.0 ** -127 and v[127] == 1.0 and v[254] == 2.0 ** 127 and np.isnan(v[255])
    if hasattr(torch, "float8_e8m0fnu"):
        t = torch.from_numpy(e[:255].copy()).view(torch.float8_e8m0fnu).double().numpy()
        assert np.array_equal(t, v[:255])


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_nvfp4_values_and_product(golden, tag):
    c, s, i = (golden[f"nvfp4_{tag}_{p}"] for p in ("codes", "scales", "inverse"))
    v = oc.nvfp4_values(c, s, i)
    assert np.array_equal(v, golden[f"nvfp4_{tag}_values"])
    x = torch.from_numpy(golden[f"nvfp4_{tag}_x"])
    assert np.array_equal(oc.gemv_exact(x, v).numpy(), golden[f"nvfp4_{tag}_exact"])
    assert np.array_equal(oc.to_blocked(s), golden[f"nvfp4_{tag}_blocked"])
    n, k = c.shape[0], c.shape[1] * 2
    assert oc.to_blocked(s).size == oc.blocked_numel(n, k)
    assert np.array_equal(oc.from_blocked(oc.to_blocked(s), n, k // 16), s)


@pytest.mark.parametrize("tag", ["row", "mx"])
def test_fp8_values_and_product(golden, tag):
    c, s = golden[f"fp8_{tag}_codes"], golden[f"fp8_{tag}_scales"]
    v = oc.fp8_values(c, s)
    assert np.array_equal(v, golden[f"fp8_{tag}_values"])
    x = torch.from_numpy(golden[f"fp8_{tag}_x"])
    assert np.array_equal(oc.gemv_exact(x, v).numpy(), golden[f"fp8_{tag}_exact"])


def test_bf16_product(golden):
    w = torch.from_numpy(golden["bf16_w"]).to(torch.bfloat16)
    x = torch.from_numpy(golden["bf16_x"])
    assert np.array_equal(oc.gemv_exact(x, oc.bf16_values(w)).numpy(), golden["bf16_exact"])


def test_generators_reproduce_the_golden_inputs(golden):
    c, s, i = wl.ref_nvfp4(96, 256)
    assert np.array_equal(c.numpy(), golden["nvfp4_a_codes"]) and np.array_equal(s.numpy(), golden["nvfp4_a_scales"])
    assert np.array_equal(i.numpy(), golden["nvfp4_a_inverse"])
    fc, fs = wl.ref_fp8(70, 512, True)
    assert np.array_equal(fc.numpy(), golden["fp8_mx_codes"]) and np.array_equal(fs.numpy(), golden["fp8_mx_scales"])
    assert np.array_equal(wl.activations(16, 256).float().numpy(), golden["nvfp4_a_x"])


@pytest.mark.parametrize("fmt", ["nvfp4", "fp8", "mxfp8", "bf16"])
def test_fp32_dequant_baseline_agrees_with_the_fp64_values(fmt):
    n, k, m = 48, 512, 4
    tensors = {"nvfp4": wl.cfg_nvfp4, "fp8": wl.cfg_fp8, "mxfp8": wl.cfg_mxfp8}.get(fmt, None)
    tensors = tensors(n, k) if tensors else (wl.cfg_bf16(n, k),)
    x = wl.activations(m, k)
    v = oc.values_of(fmt, tensors)
    deq = oc.dequant_fp32(fmt, tensors)
    if fmt == "fp8":      # code * FP32 row scale rounds once in FP32
        assert np.allclose(deq.double().numpy(), v, rtol=1e-7, atol=0)
    else:                 # code * block scale (* inverse 1.0) is exact in FP32
        assert np.array_equal(deq.double().numpy(), v)
    out = oc.gemv_fp32(x, deq, torch.float32)
    assert oc.within_fp32_bound(out, x, v)
    assert oc.max_rel_error(oc.gemv_fp32(x, deq), oc.gemv_exact(x, v)) < 1e-2


def test_mxfp8_generator_follows_the_shared_exponent_rule():
    c, e = wl.cfg_mxfp8(8, 256)
    v = oc.e4m3_to_float(c.numpy()).reshape(8, -1, 32)
    assert not np.isnan(v).any()
    amax = np.abs(v).max(axis=-1)
    assert (amax >= 256).all() and (amax <= 448).all()      # block max scaled into [256, 512), saturated at 448
    assert e.min() > 90 and e.max() < 130


def test_weight_bytes_of_the_configurations():
    assert wl.weight_bytes("nvfp4", 4096, 4096) == 9_453_568
    assert wl.weight_bytes("fp8", 28672, 8192) == 234_995_712
    assert wl.weight_bytes("mxfp8", 13824, 5120) == 72_990_720
    assert wl.weight_bytes("bf16", 8192, 8192) == 134_217_728
    assert sum(wl.weight_bytes("nvfp4", n, k) for _, k, n in wl.STACK_ROLES) == 481_632_256


# ----- the dequantizers -------------------------------------------------------------------------------------------

@pytest.mark.parametrize("tag", ["a", "b"])
def test_dequantize_matches_the_reference_tests_expectation(golden, tag):
    """oracle.dequantize against what decode-gemv/tests/test_decode_gemv.py:131-140 expects of decode / decode_fp8
    (golden vectors made from that expression on the reference's own generators)."""
    g = golden
    c, s, i = g[f"nvfp4_{tag}_codes"], g[f"nvfp4_{tag}_scales"], g[f"nvfp4_{tag}_inverse"]
    bf = oc.dequantize(c, s, i, torch.bfloat16)
    assert np.array_equal(bf.view(torch.int16).numpy(), g[f"nvfp4_{tag}_decode_bf16"])
    fp = oc.dequantize(c, s, i, torch.float16)
    assert np.array_equal(fp.view(torch.int16).numpy(), g[f"nvfp4_{tag}_decode_f16"])
    f8 = oc.dequantize(c, s, i * np.float32(64), torch.float8_e4m3fn)
    assert np.array_equal(f8.view(torch.uint8).numpy(), g[f"nvfp4_{tag}_decode_fp8"])


def test_dequantize_saturates_and_rounds_once():
    codes = np.array([[0x77, 0xF7, 0x21, 0x00, 0x10, 0x01, 0x99, 0xAB]], dtype=np.uint8)     # 16 values, one block
    scales = np.array([[0x7E]], dtype=np.uint8)                                                # E4M3 448
    out = oc.dequantize(codes, scales, np.array([1.0], dtype=np.float32), torch.float8_e4m3fn).float().numpy()
    assert out.max() == 448.0 and out.min() == -448.0                                          # 6 * 448 clamps
    third = np.array([1.0 / 3.0], dtype=np.float32)
    bf = oc.dequantize(codes, np.array([[0x38]], dtype=np.uint8), third, torch.bfloat16)      # scale 1.0
    want = torch.from_numpy(oc.nvfp4_values(codes, np.array([[0x38]], dtype=np.uint8), np.ones(1, np.float32))
                            .astype(np.float32) * third[:, None]).to(torch.bfloat16)
    assert torch.equal(bf, want)


# ----- the reference's C++ host oracle (row_fp8.h, fp8_block.h) ---------------------------------------------------

def test_e4m3_decode_matches_the_reference_host_oracle(golden):
    """crit::fp8::decode (fp8-block-rows/tests/order/row_fp8.h:25-31) for every byte it accepts."""
    mine = oc.e4m3_to_float(np.arange(256, dtype=np.uint8))
    want = golden["host_decode"].astype(np.float64)
    ok = ~np.isnan(want)
    assert ok.sum() == 254 and np.array_equal(mine[ok], want[ok])
    assert np.array_equal(np.signbit(mine[ok]), np.signbit(want[ok])) and np.isnan(mine[~ok]).all()


def test_fp8_projection_matches_the_reference_host_oracle(golden):
    """crit::fp8::project (row_fp8.h:86-98): FP64 projection of E4M3 codes with BF16 row scales and BF16 activations,
    against the Python oracle's stored values and exact product (summation order differs: 1e-12)."""
    def bf16(words):
        return torch.from_numpy(words.astype(np.int16)).view(torch.bfloat16)
    codes = golden["host_codes"]
    scales = bf16(golden["host_scales_bf16"]).float()
    x = bf16(golden["host_x_bf16"])
    mine = oc.gemv_exact(x, oc.fp8_values(codes, scales)).numpy()
    want = golden["host_project"]
    assert np.allclose(mine, want, rtol=1e-12, atol=1e-300)


def test_mx_groups_match_the_reference_host_quantizer(golden):
    """crit::fp8_block::quantize_group, MX kind (fp8_block.h:24-39): the shared exponent and the E4M3 codes of the
    workload generator's MXFP8 groups, and e8m0 (fp8_block.h:18-21) against the oracle's E8M0 decode."""
    values = torch.from_numpy(golden["host_mx_values"])
    codes, mx = wl.mx_quantize(values)
    scale = oc.e8m0_to_float(mx.numpy())
    assert np.array_equal(scale, golden["host_mx_scale"].astype(np.float64))
    assert np.array_equal(scale, golden["host_mx_e8m0"].astype(np.float64))
    assert np.array_equal(codes.numpy() & 127, golden["host_mx_codes"] & 127)                 # magnitudes
    nonzero = (golden["host_mx_codes"] & 127) != 0
    assert np.array_equal((codes.numpy() & 128)[nonzero], (golden["host_mx_codes"] & 128)[nonzero])


def test_quantizer_oracle_reproduces_the_reference_tests_quantizers():
    """tests/golden/quantize_golden.npz holds what the reference test's own torch quantizers (mma-rows/tests/
    test_mma_rows.py:80-104) give on its own inputs, evaluated on a B200 by tests/golden/make_quantize_golden.py."""
    import os
    import numpy as np
    import torch
    from oracle import quantize_oracle as qo
    from oracle import decode_gemv_oracle as oc
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "quantize_golden.npz"))
    scale_in = float(g["input_scale"])
    for tag in ("a", "c"):
        x = torch.from_numpy(g[f"{tag}_x"]).view(torch.bfloat16)
        q, scale = qo.fp8_rows(x)
        assert np.array_equal(q, g[f"{tag}_q"]), tag
        assert np.array_equal(scale.view(np.uint32), g[f"{tag}_scale"].view(np.uint32)), tag
        codes, sbits = qo.nvfp4(x, scale_in)
        assert np.array_equal(codes, g[f"{tag}_codes"]), tag
        assert np.array_equal(sbits, g[f"{tag}_block_scales"]), tag
    assert np.array_equal(qo.nvfp4_blocked(torch.from_numpy(g["a_x"]).view(torch.bfloat16), scale_in)[1], g["a_blocked"])
    assert np.array_equal(oc.to_blocked(g["a_block_scales"]), g["a_blocked"])
    xb = torch.from_numpy(g["b_x"]).view(torch.bfloat16)
    for k in (1001, 20000):
        q, scale = qo.fp8_rows(xb[:, :k])
        assert np.array_equal(q, g[f"b_q_{k}"]) and np.array_equal(scale, g[f"b_scale_{k}"]), k
