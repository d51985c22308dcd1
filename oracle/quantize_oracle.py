"""TEST INFRASTRUCTURE ONLY: CPU restatement of the reference's activation quantizers, the checker of
crit_kernels_b200/csrc/dg_quantize.cu. Nothing shipped imports this module.

What it restates, operation for operation in FP32 (numpy float32 arithmetic is IEEE, like the kernels' __fdiv_rn and
plain multiplies):
  * quantize_fp8_rows  mma-rows/mma_rows_cuda/mma_rows.cu:15-90 with tile_parts.cuh:23-25 (fp32(1 / 448) as a factor),
                       :35 (nanmax), :42-44 (E4M3, nearest even, saturating), :301-305 (fp8_value)
  * quantize_nvfp4     mma_rows.cu:117-140 with tile_parts.cuh:57-64 (e2m1_code: thresholds 0.25 ... 5, ties to the even
                       code, sign bit for v < 0) and :309-331 (nvfp4_block: block scale, divisor, the zero rule)
The reference's tests state the same quantizers as torch expressions on CUDA tensors (mma-rows/tests/
test_mma_rows.py:80-104); torch divides a CUDA tensor by a Python constant as a product with the constant's FP32
reciprocal, which is why the kernels and this file multiply by fp32(1 / 448) and fp32(1 / 6) (on CPU tensors torch
divides, so those expressions are evaluated on the GPU box: tests/golden/make_quantize_golden.py).

Pinned by tests/golden/quantize_golden.npz (outputs of the reference test's own functions on its own inputs, evaluated
on a B200) and, on a GPU box, bit for bit against the reference's kernels built into oracle/_ref/libmma_rows_ref.so.
"""
from __future__ import annotations

import numpy as np
import torch

from .decode_gemv_oracle import e4m3_to_float, to_blocked

RCP448 = np.float32(1.0) / np.float32(448.0)
RCP6 = np.float32(1.0) / np.float32(6.0)


def _f32(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().float().numpy()
    return np.asarray(x, dtype=np.float32)


def _e4m3_bits(v: np.ndarray) -> np.ndarray:
    """FP32 (already within +-448, or NaN) -> E4M3 bytes, round to nearest even (torch's cast does exactly that)."""
    return torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def fp8_rows(x):
    """x [M][K] BF16 -> (q uint8 [M][K], scale float32 [M])."""
    v = _f32(x)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        amax = np.max(np.abs(v), axis=1).astype(np.float32)            # NaN if the row holds one (nanmax)
        scale = (amax * RCP448).astype(np.float32)
        scale = np.where(scale < np.float32(1e-12), np.float32(1e-12), scale).astype(np.float32)
        r = (v / scale[:, None]).astype(np.float32)
        r = np.where(r > 448, np.float32(448), np.where(r < -448, np.float32(-448), r)).astype(np.float32)
    return _e4m3_bits(r), scale


def nvfp4(x, input_scale):
    """x [M][K] BF16, K % 16 == 0 -> (codes uint8 [M][K / 2], block scale bytes uint8 [M][K / 16])."""
    v = _f32(x)
    m, k = v.shape
    g = np.float32(input_scale)
    g_rcp = np.float32(1.0) / g
    blocks = v.reshape(m, k // 16, 16)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        amax = np.max(np.abs(blocks), axis=2).astype(np.float32)
        bs = ((amax * RCP6).astype(np.float32) * g).astype(np.float32)
        bs = np.where(bs > 448, np.float32(448), bs).astype(np.float32)
        sbits = _e4m3_bits(bs)
        d = (e4m3_to_float(sbits).astype(np.float32) * g_rcp).astype(np.float32)
        zero = ~(d > 0)
        d = np.where(d < np.float32(1e-30), np.float32(1e-30), d).astype(np.float32)
        q = (blocks / d[..., None]).astype(np.float32)
        q = np.where(zero[..., None], np.float32(0), q)
        mag = np.abs(q)
        mag = np.where(mag > 6, np.float32(6), mag)
        code = np.zeros(mag.shape, dtype=np.uint8)
        for bound in (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0):
            code += (mag > np.float32(bound)).astype(np.uint8)
        code += ((mag == 0.75) | (mag == 1.75) | (mag == 3.5)).astype(np.uint8)
        code |= (q < 0).astype(np.uint8) << 3
    code = code.reshape(m, k)
    return (code[:, 0::2] | (code[:, 1::2] << 4)).astype(np.uint8), sbits


def nvfp4_blocked(x, input_scale):
    """As nvfp4, the scales in the 128 x 4 tiled layout (flat, padding zero) the kernels write."""
    codes, sbits = nvfp4(x, input_scale)
    return codes, to_blocked(sbits)
