"""Decode GEMVs for B200, weight only: NVFP4 weights (W4A16), FP8 E4M3 weights with a row scale or MXFP8's E8M0 scale
per 32 inputs (W8A16) and BF16 weights, times 1 to 16 rows of 16-bit activations, on CUDA cores with FP32 sums. Each
row's result is the same bits alone and beside the other rows of a call, and the same bits from any slice of the
matrix's rows: the summation order depends on K and the format only.

Same functions, argument layouts and refusals as the reference package's CUDA entry points
(decode-gemv/torch-ext/decode_gemv/__init__.py:19-53), plus the NVFP4 dequantizers decode and decode_fp8, which the
reference implements in Triton (triton_gemv.py:171-200) and this package in CUDA. The reference's other Triton entry
points (gemv_triton, gemv_fp8_dot, ...) are not part of this package.

NVFP4 matrices as checkpoints store them: codes [N][K / 2] uint8 (element 2i in the low nibble of byte i), E4M3 block
scales [N][K / 16] (row major, or cuBLASLt's 128 x 4 tiles with blocked=True) and inverse [N] FP32 (one over each row's
global scale). FP8: codes [N][K] E4M3 and FP32 row scales [N], or E8M0 bytes [N][K / 32] (MXFP8)."""
import torch

from ._ops import ops

CUDA_ROWS = 16   # rows the GEMVs take in one call

__all__ = ["CUDA_ROWS", "gemv", "gemv_fp8", "gemv_bf16", "hardware_decode", "decode", "decode_fp8"]

_TRITON_SIDE = {"DOT_ROWS", "TRITON_ROWS", "dot_partial_elements", "fp8_dot_tile", "gemv_fp8_dot", "gemv_triton",
                "hardware"}


def gemv(x: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, inverse: torch.Tensor, out: torch.Tensor,
         blocked: bool = False):
    """out [M][N] (FP32 or x's dtype) = x [M][K] (M 1..16, BF16 or FP16, rows on 16-byte boundaries, K a multiple of
    32) times the NVFP4 matrix. blocked: the E4M3 block scales are in cuBLASLt's 128 x 4 tiled layout (rows padded to
    128, blocks to 4) instead of row major [N][K / 16]. Returns out."""
    ops.gemv(x, codes, scales, inverse, blocked, out)
    return out


def gemv_fp8(x: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, out: torch.Tensor):
    """out [M][N] (FP32 or x's dtype) = x [M][K] (M 1..16, BF16 or FP16) times the FP8 matrix: codes [N][K] E4M3
    (float8_e4m3fn or uint8, K a multiple of 16) with scales FP32 [N] (one per row, applied after the sum) or uint8
    E8M0 [N][K / 32] (MXFP8, each value times its power of two). Returns out."""
    ops.gemv_fp8(x, codes.view(torch.uint8), scales, out)
    return out


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
    """out [M][N] (FP32 or BF16) = x [M][K] (M 1..16, BF16) times w [N][K] BF16 (K a multiple of 8). Returns out."""
    ops.gemv_bf16(x, w, out)
    return out


def hardware_decode(device=None) -> bool:
    """Whether the GEMV's code for `device` decodes E2M1 by the hardware conversion: always, on the sm_100a target
    this package is built for."""
    device = torch.device(device or "cuda")
    return bool(ops.hardware_decode(torch.empty(0, device=device)))


def decode(codes: torch.Tensor, scales: torch.Tensor, inverse: torch.Tensor, out: torch.Tensor):
    """The NVFP4 matrix's values [N][K] in out's dtype (BF16 or FP16, contiguous): e2m1 * scale * inverse, one FP32
    product rounded once. codes [N][K / 2] uint8, scales [N][K / 16] E4M3 (row major), inverse [N] FP32. Returns
    out."""
    if out.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"decode: out must be BF16 or FP16, got {out.dtype} (decode_fp8 writes FP8 E4M3)")
    ops.decode(codes, scales, inverse, out)
    return out


def decode_fp8(codes: torch.Tensor, scales: torch.Tensor, factor: torch.Tensor, out: torch.Tensor):
    """The NVFP4 matrix's values [N][K] as FP8 E4M3 (out contiguous float8_e4m3fn) in units of each row's scale: e2m1 *
    scale * factor[row], rounded once to nearest even within +-448. Returns out."""
    if out.dtype != torch.float8_e4m3fn:
        raise RuntimeError(f"decode_fp8: out must be float8_e4m3fn, got {out.dtype}")
    ops.decode(codes, scales, factor, out)
    return out


def __getattr__(name):
    if name in _TRITON_SIDE:
        raise AttributeError(f"decode_gemv.{name} is one of the reference's Triton entry points; this B200 package "
                             "provides CUDA kernels only (gemv, gemv_fp8, gemv_bf16, hardware_decode, decode, decode_fp8)")
    raise AttributeError(name)
