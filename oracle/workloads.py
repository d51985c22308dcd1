"""Seeded synthetic inputs for the decode-gemv configurations. TEST / BENCH INFRASTRUCTURE ONLY (see
decode_gemv_oracle.py): these generators stand in for real checkpoints, which the reference's own tests do not use
either (decode-gemv/tests/test_decode_gemv.py:20-26, 37-38, 198-207 draw everything from seeded generators).

Two families:
  * `ref_*`   the distributions of the reference's tests (uniform codes, scales in (0.01, 4.01), ...), used by the
              parity tests so they read like the reference's;
  * `cfg_*`   the distributions the benchmark configurations name (E4M3 casts of N(0, 0.02) weights, power-of-two-ish
              NVFP4 block scales, the MX shared-exponent rule 2^(floor(log2 amax) - 8) of
              fp8-block-rows/tests/order/fp8_block.h:24-39).
All tensors are created on the CPU from torch.Generator().manual_seed(seed).
"""
from __future__ import annotations

import torch


def _gen(seed):
    return torch.Generator().manual_seed(int(seed))


def activations(m, k, dtype=torch.bfloat16, seed=8):
    """randn [M][K] rounded to dtype (test_decode_gemv.py:37-38)."""
    return torch.randn(m, k, generator=_gen(seed)).to(dtype)


# ----- the reference tests' distributions ------------------------------------------------------------------------

def ref_nvfp4(n, k, seed=5):
    """codes uint8 [N][K/2], E4M3 scales [N][K/16] as uint8 bytes, inverse FP32 [N] (test_decode_gemv.py:20-26)."""
    g = _gen(seed)
    codes = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    scales = (torch.rand(n, k // 16, generator=g) * 4 + 0.01).to(torch.float8_e4m3fn)
    inverse = (torch.rand(n, generator=g) + 0.5) / 64
    return codes, scales.view(torch.uint8), inverse


def ref_fp8(n, k, mx, seed=6):
    """E4M3 codes without NaN and FP32 row scales, or E8M0 exponents in [118, 132) (test_decode_gemv.py:198-207)."""
    g = _gen(seed)
    codes = torch.randint(0, 0x7E, (n, k), generator=g, dtype=torch.uint8)
    codes = codes | (torch.randint(0, 2, (n, k), generator=g, dtype=torch.uint8) << 7)
    if mx:
        scales = torch.randint(118, 132, (n, k // 32), generator=g, dtype=torch.uint8)
    else:
        scales = torch.rand(n, generator=g) / 100 + 1e-3
    return codes, scales


def ref_bf16(n, k, seed=3, std=0.05):
    return (torch.randn(n, k, generator=_gen(seed)) * std).to(torch.bfloat16)


# ----- the benchmark configurations' distributions ----------------------------------------------------------------

def cfg_nvfp4(n, k, seed=0):
    """Uniform E2M1 codes, E4M3 block scales nearest 2^u with u ~ U(-4, 2), global scale 1 (inverse = ones)."""
    g = _gen(seed)
    codes = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8)
    scales = torch.exp2(torch.rand(n, k // 16, generator=g) * 6 - 4).to(torch.float8_e4m3fn)
    return codes, scales.view(torch.uint8), torch.ones(n)


def cfg_fp8(n, k, seed=1):
    """E4M3 casts of N(0, 0.02) weights; row scales U(0.5, 2) * 2^-6."""
    g = _gen(seed)
    codes = (torch.randn(n, k, generator=g) * 0.02).to(torch.float8_e4m3fn).view(torch.uint8)
    scales = (torch.rand(n, generator=g) * 1.5 + 0.5) / 64
    return codes, scales


def mx_shared_exponent(amax):
    """The MX shared exponent of groups with these maxima: floor(log2(amax)) - 8, 0 for an all-zero group, kept in
    [-127, 127]: the reference's rule (fp8-block-rows/tests/order/fp8_block.h:28-33, frexp(amax) - 1 - 8)."""
    _, e = torch.frexp(amax.float())                       # amax = m * 2^e with m in [0.5, 1)
    shared = torch.where(amax > 0, e - 1 - 8, torch.zeros_like(e))
    return shared.clamp(-127, 127).float()


def mx_quantize(w):
    """[..., 32] FP32 groups -> (E4M3 codes as uint8 [..., 32], E8M0 bytes [...]): codes = E4M3(w / 2^shared), nearest
    even, saturating at +-448 (a torch cast above 448 would give NaN, hence the clamp)."""
    shared = mx_shared_exponent(w.abs().amax(dim=-1))
    codes = (w / torch.exp2(shared)[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return codes.view(torch.uint8), (shared + 127).to(torch.uint8)


def cfg_mxfp8(n, k, seed=2):
    """MXFP8 of N(0, 0.02) weights: per 32 inputs shared = floor(log2(amax)) - 8, byte = shared + 127, codes =
    E4M3(w / 2^shared)."""
    g = _gen(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).view(n, k // 32, 32)
    codes, mx = mx_quantize(w)
    return codes.view(n, k), mx


def cfg_bf16(n, k, seed=3):
    return (torch.randn(n, k, generator=_gen(seed)) * 0.02).to(torch.bfloat16)


# The 70B-shaped decode projection stack: (role, K, N) per layer, 80 layers.
STACK_ROLES = (("qkv", 8192, 10240), ("o", 8192, 8192), ("gate_up", 8192, 57344), ("down", 28672, 8192))
STACK_LAYERS = 80


def weight_bytes(fmt, n, k) -> int:
    """Algorithmic weight bytes one call streams: codes + block scales + per-row scales."""
    if fmt == "nvfp4":
        return n * k // 2 + n * k // 16 + 4 * n
    if fmt == "fp8":
        return n * k + 4 * n
    if fmt == "mxfp8":
        return n * k + n * k // 32
    if fmt == "bf16":
        return 2 * n * k
    raise ValueError(fmt)
