// Torch entry points of the B200 decode GEMVs: the op surface of the reference package decode-gemv
// (decode-gemv/torch-ext/torch_binding.h:8-16), same argument order and meaning.
#pragma once

#include <torch/types.h>

// x [M][K] (M 1..16) BF16 or FP16; codes [N][K / 2] uint8; scales E4M3 bytes, row major [N][K / 16] or, blocked,
// cuBLASLt's 128 x 4 tiles; inverse [N] FP32; out [M][N] FP32 or x's dtype.
void gemv(const torch::Tensor& x, const torch::Tensor& codes, const torch::Tensor& scales,
          const torch::Tensor& inverse, bool blocked, torch::Tensor& out);
// x as above; codes [N][K] E4M3 bytes; scales FP32 [N] (row scales) or uint8 [N][K / 32] (MXFP8 exponents).
void gemv_fp8(const torch::Tensor& x, const torch::Tensor& codes, const torch::Tensor& scales, torch::Tensor& out);
// x [M][K] BF16; w [N][K] BF16; out FP32 or BF16.
void gemv_bf16(const torch::Tensor& x, const torch::Tensor& w, torch::Tensor& out);
// 1: E2M1 decodes by the hardware conversion on device_of's device (always, for this sm_100a build).
int64_t hardware_decode(const torch::Tensor& device_of);
// The NVFP4 matrix's values into out [N][K] (contiguous BF16, FP16 or FP8 E4M3): e2m1 * scale * factor[row], one FP32
// product rounded once (FP8: saturating at +-448). codes [N][K / 2] uint8, scales [N][K / 16] E4M3 bytes, factor [N]
// FP32. The reference's decode and decode_fp8 (decode-gemv/torch-ext/decode_gemv/triton_gemv.py:171-176, :195-200).
void decode(const torch::Tensor& codes, const torch::Tensor& scales, const torch::Tensor& factor, torch::Tensor& out);
// Activation quantizers (the reference's mma-rows package, mma-rows/torch-ext/torch_binding.h): x [rows][K] BF16, any
// number of rows. FP8 per row: q [rows][K] E4M3 bytes, scale [rows] FP32. NVFP4: codes [rows][K / 2] bytes and E4M3
// block scales in 128 x 4 tiles (rows padded to 128, blocks to 4) under input_scale.
void quantize_fp8_rows(const torch::Tensor& x, torch::Tensor& q, torch::Tensor& scale);
void quantize_nvfp4(const torch::Tensor& x, double input_scale, torch::Tensor& codes, torch::Tensor& scales);
