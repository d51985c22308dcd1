"""Weight-only decode projections for B200: y = x W^T for 1 to 16 activation rows x (BF16 or FP16) and a weight matrix
W kept in its checkpoint format: NVFP4 (4-bit E2M1 codes with an E4M3 scale per 16 inputs), FP8 E4M3 with one FP32
scale per output channel, MXFP8 (E4M3 with a power-of-two E8M0 scale per 32 inputs) or plain BF16. The products are
summed in FP32 on CUDA cores in an order that depends only on K and the format, so an output row has the same bits
whether it is computed alone, among other rows, or from a slice of W's rows on another GPU.

This module is what `get_kernel("crit-labs/decode-gemv")` hands out: `gemv`, `gemv_fp8`, `gemv_bf16`,
`hardware_decode` and `CUDA_ROWS` take the arguments of the reference package's functions of those names
(decode-gemv/torch-ext/decode_gemv/__init__.py:19-53) and refuse what they refuse. Beyond that surface it carries the
pieces either side of the GEMVs that the reference keeps elsewhere: `decode` / `decode_fp8` (its Triton dequantizers,
triton_gemv.py:171-200, here in CUDA) and `quantize_fp8_rows` / `quantize_nvfp4` (the activation quantizers of its
mma-rows package). The reference's Triton GEMVs (gemv_triton, gemv_fp8_dot and their helpers) have no counterpart here.

Storage: NVFP4 codes [N][K / 2] uint8 with input 2i in the low nibble of byte i, block scales [N][K / 16] E4M3 either
row major or, with blocked=True, in cuBLASLt's 128 x 4 tiles, and inverse [N] FP32 = 1 / the row's global scale; FP8
codes [N][K] with FP32 scales [N], or with E8M0 bytes [N][K / 32] for MXFP8."""
import torch

from ._ops import ops

CUDA_ROWS = 16   # rows the GEMVs take in one call

__all__ = ["CUDA_ROWS", "gemv", "gemv_fp8", "gemv_bf16", "hardware_decode", "decode", "decode_fp8", "quantize_fp8_rows",
           "quantize_nvfp4"]

_TRITON_SIDE = {"DOT_ROWS", "TRITON_ROWS", "dot_partial_elements", "fp8_dot_tile", "gemv_fp8_dot", "gemv_triton",
                "hardware"}


def gemv(x: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, inverse: torch.Tensor, out: torch.Tensor,
         blocked: bool = False):
    """NVFP4 projection. Writes x @ W^T into out and returns it. x: [M][K], 1 <= M <= 16, BF16 or FP16, every row on
    a 16-byte boundary, K % 32 == 0. out: [M][N], FP32 or x's dtype. Pass blocked=True when `scales` uses the
    128 x 4 tiled layout (128-row, 4-block padding) rather than plain [N][K / 16]."""
    ops.gemv(x, codes, scales, inverse, blocked, out)
    return out


def gemv_fp8(x: torch.Tensor, codes: torch.Tensor, scales: torch.Tensor, out: torch.Tensor):
    """FP8 projection. Writes x @ W^T into out and returns it. codes: [N][K] E4M3 (float8_e4m3fn or raw uint8),
    K % 16 == 0. The dtype of `scales` picks the flavour: FP32 [N] multiplies each finished sum by its channel's
    scale; uint8 [N][K / 32] are MXFP8 exponents, each weight counting 2^(e - 127) times its code (K % 32 == 0)."""
    ops.gemv_fp8(x, codes.view(torch.uint8), scales, out)
    return out


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
    """BF16 projection, the pure bandwidth case. x [M][K] and w [N][K] BF16, K % 8 == 0; out [M][N] FP32 or BF16,
    returned."""
    ops.gemv_bf16(x, w, out)
    return out


def hardware_decode(device=None) -> bool:
    """True when E2M1 codes are decoded by the conversion instruction rather than by bit arithmetic on `device`.
    This build targets sm_100a only, where that is always so; a device it cannot run on raises RuntimeError."""
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


def quantize_fp8_rows(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor):
    """BF16 rows to FP8: q [rows][K] (float8_e4m3fn or uint8) = x / scale rounded to E4M3, with scale [rows] FP32 =
    max(|row|) / 448 (at least 1e-12) written too. Any number of rows and any K. The arithmetic and bits of the
    reference's mma_rows.quantize_fp8_rows (mma-rows/torch-ext/mma_rows/__init__.py:124-128). Returns (q, scale)."""
    ops.quantize_fp8_rows(x, q.view(torch.uint8), scale)
    return q, scale


def quantize_nvfp4(x: torch.Tensor, input_scale: float, codes: torch.Tensor, scales: torch.Tensor):
    """BF16 rows to NVFP4 under `input_scale`: codes [rows][K / 2] (two E2M1 codes a byte, the even input low) and one
    E4M3 scale per 16 inputs, stored in 128 x 4 tiles with rows padded to 128 and blocks to 4 (padding zeroed).
    K % 16 == 0. The bits of the reference's mma_rows.quantize_nvfp4 (mma-rows/torch-ext/mma_rows/__init__.py:131-136).
    Returns (codes, scales)."""
    ops.quantize_nvfp4(x, float(input_scale), codes.view(torch.uint8), scales.view(torch.uint8))
    return codes, scales


def __getattr__(name):
    if name in _TRITON_SIDE:
        raise AttributeError(f"decode_gemv.{name} is one of the reference's Triton entry points; this B200 package "
                             "provides CUDA kernels only (gemv, gemv_fp8, gemv_bf16, hardware_decode, decode, decode_fp8)")
    raise AttributeError(name)
