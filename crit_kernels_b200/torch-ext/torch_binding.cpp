// Torch op registration and argument checks over the C ABI (include/decode_gemv_b200.h).
//
// The GEMV schemas are those of the reference (decode-gemv/torch-ext/torch_binding.cpp:7-10; `decode`, the NVFP4
// dequantizer, is a Triton function there and an op only here), CUDA implementations only,
// and every refusal of its entry points (decode-gemv/decode_gemv_cuda/binding.cu:19-118) is kept: a violated rule
// raises c10::Error, a Python RuntimeError. Nothing here allocates or waits for the device, and the launch goes to
// the current stream of x's device, so a CUDA graph captures the calls.
#include "torch_binding.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime_api.h>
#include <torch/library.h>

#include <cstdint>

#include "../../include/decode_gemv_b200.h"

#ifndef DG_TORCH_NAMESPACE
#define DG_TORCH_NAMESPACE _decode_gemv_b200
#endif

namespace {

bool on_boundary(const torch::Tensor& t, std::uintptr_t bytes) {
  return reinterpret_cast<std::uintptr_t>(t.data_ptr()) % bytes == 0;
}

// x: 2-D CUDA, 1..16 rows, unit inner stride, rows 16 bytes apart on a 16-byte base; BF16, or FP16 where allowed.
void require_activations(const torch::Tensor& x, bool fp16_ok, const char* op) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2, op, ": x must be a 2-D CUDA tensor [rows][K]");
  TORCH_CHECK(x.size(0) >= 1 && x.size(0) <= DG_MAX_ROWS, op, ": x has ", x.size(0), " rows; 1 to ", DG_MAX_ROWS,
              " are supported");
  TORCH_CHECK(x.stride(1) == 1 && x.stride(0) % 8 == 0 && on_boundary(x, 16), op,
              ": rows of x must be contiguous and start on 16-byte boundaries");
  if (fp16_ok) {
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16 || x.scalar_type() == torch::kFloat16, op,
                ": x must be BF16 or FP16");
  } else {
    TORCH_CHECK(x.scalar_type() == torch::kBFloat16, op, ": x must be BF16");
  }
}

void require_output(const torch::Tensor& out, const torch::Tensor& x, int64_t n, const char* op) {
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.size(0) == x.size(0) && out.size(1) == n && out.stride(1) == 1,
              op, ": out must be [rows][N] with contiguous rows");
  TORCH_CHECK(out.scalar_type() == torch::kFloat32 || out.scalar_type() == x.scalar_type(), op,
              ": out must be FP32 or have x's dtype");
}

void require_same_device(const torch::Tensor& x, std::initializer_list<const torch::Tensor*> rest, const char* op) {
  for (const torch::Tensor* t : rest)
    TORCH_CHECK(t->device() == x.device(), op, ": all tensors must be on x's device (", x.device(), "), found ",
                t->device());
}

void require_success(int code, const char* op) {
  TORCH_CHECK(code == 0, op, ": ", cudaGetErrorString(static_cast<cudaError_t>(code)));
}

}  // namespace

void gemv(const torch::Tensor& x, const torch::Tensor& codes, const torch::Tensor& scales,
          const torch::Tensor& inverse, bool blocked, torch::Tensor& out) {
  const char* op = "gemv";
  require_activations(x, true, op);
  const int64_t n = codes.size(0), k = x.size(1);
  TORCH_CHECK(k % 32 == 0, op, ": K must be a multiple of 32, got ", k);
  TORCH_CHECK(codes.is_cuda() && codes.dim() == 2 && codes.is_contiguous() && codes.scalar_type() == torch::kUInt8 &&
                  codes.size(1) * 2 == k && on_boundary(codes, 16),
              op, ": codes must be contiguous uint8 [N][K / 2] on a 16-byte boundary");
  TORCH_CHECK(scales.is_cuda() && scales.is_contiguous() && scales.element_size() == 1 && on_boundary(scales, 2), op,
              ": scales must be contiguous E4M3 bytes on a 2-byte boundary");
  if (blocked) {
    TORCH_CHECK(scales.numel() == ((n + 127) / 128) * 128 * ((k / 16 + 3) / 4) * 4, op,
                ": blocked scales must hold the 128 x 4 tiles of [N][K / 16] (rows padded to 128, blocks to 4)");
  } else {
    TORCH_CHECK(scales.dim() == 2 && scales.size(0) == n && scales.size(1) * 16 == k, op,
                ": scales must be E4M3 bytes [N][K / 16]");
  }
  TORCH_CHECK(inverse.is_cuda() && inverse.is_contiguous() && inverse.scalar_type() == torch::kFloat32 &&
                  inverse.numel() == n && on_boundary(inverse, 4),
              op, ": inverse must be contiguous FP32 [N]");
  require_output(out, x, n, op);
  require_same_device(x, {&codes, &scales, &inverse, &out}, op);
  const c10::cuda::CUDAGuard guard(x.device());
  require_success(dg_enqueue_nvfp4(x.data_ptr(), static_cast<int>(x.stride(0)), x.scalar_type() == torch::kBFloat16,
                                   codes.data_ptr<std::uint8_t>(), static_cast<const std::uint8_t*>(scales.data_ptr()),
                                   blocked, inverse.data_ptr<float>(), out.data_ptr(), static_cast<int>(out.stride(0)),
                                   out.scalar_type() == torch::kFloat32 ? 0 : 1, static_cast<int>(x.size(0)),
                                   static_cast<int>(n), static_cast<int>(k), at::cuda::getCurrentCUDAStream().stream()),
                  op);
}

void gemv_fp8(const torch::Tensor& x, const torch::Tensor& codes, const torch::Tensor& scales, torch::Tensor& out) {
  const char* op = "gemv_fp8";
  require_activations(x, true, op);
  const int64_t n = codes.size(0), k = x.size(1);
  TORCH_CHECK(codes.is_cuda() && codes.dim() == 2 && codes.is_contiguous() && codes.element_size() == 1 &&
                  codes.size(1) == k && k % 16 == 0 && on_boundary(codes, 16),
              op, ": codes must be contiguous E4M3 bytes [N][K] on a 16-byte boundary, K a multiple of 16");
  TORCH_CHECK(scales.is_cuda() && scales.is_contiguous(), op, ": scales must be a contiguous CUDA tensor");
  const bool mx = scales.scalar_type() == torch::kUInt8;
  if (mx) {
    TORCH_CHECK(scales.dim() == 2 && scales.size(0) == n && k % 32 == 0 && scales.size(1) * 32 == k, op,
                ": MXFP8 scales must be E8M0 bytes [N][K / 32], K a multiple of 32");
  } else {
    TORCH_CHECK(scales.scalar_type() == torch::kFloat32 && scales.numel() == n && on_boundary(scales, 4), op,
                ": row scales must be FP32 [N] (or uint8 E8M0 [N][K / 32] for MXFP8)");
  }
  require_output(out, x, n, op);
  require_same_device(x, {&codes, &scales, &out}, op);
  const c10::cuda::CUDAGuard guard(x.device());
  require_success(dg_enqueue_fp8(x.data_ptr(), static_cast<int>(x.stride(0)), x.scalar_type() == torch::kBFloat16,
                                 static_cast<const std::uint8_t*>(codes.data_ptr()),
                                 mx ? nullptr : scales.data_ptr<float>(),
                                 mx ? scales.data_ptr<std::uint8_t>() : nullptr, out.data_ptr(),
                                 static_cast<int>(out.stride(0)), out.scalar_type() == torch::kFloat32 ? 0 : 1,
                                 static_cast<int>(x.size(0)), static_cast<int>(n), static_cast<int>(k),
                                 at::cuda::getCurrentCUDAStream().stream()),
                  op);
}

void gemv_bf16(const torch::Tensor& x, const torch::Tensor& w, torch::Tensor& out) {
  const char* op = "gemv_bf16";
  require_activations(x, false, op);
  const int64_t n = w.size(0), k = x.size(1);
  TORCH_CHECK(w.is_cuda() && w.dim() == 2 && w.is_contiguous() && w.scalar_type() == torch::kBFloat16 &&
                  w.size(1) == k && k % 8 == 0 && on_boundary(w, 16),
              op, ": w must be contiguous BF16 [N][K] on a 16-byte boundary, K a multiple of 8");
  require_output(out, x, n, op);
  require_same_device(x, {&w, &out}, op);
  const c10::cuda::CUDAGuard guard(x.device());
  require_success(dg_enqueue_bf16(x.data_ptr(), static_cast<int>(x.stride(0)), w.data_ptr(), out.data_ptr(),
                                  static_cast<int>(out.stride(0)), out.scalar_type() == torch::kFloat32 ? 0 : 1,
                                  static_cast<int>(x.size(0)), static_cast<int>(n), static_cast<int>(k),
                                  at::cuda::getCurrentCUDAStream().stream()),
                  op);
}

void decode(const torch::Tensor& codes, const torch::Tensor& scales, const torch::Tensor& factor,
            torch::Tensor& out) {
  const char* op = "decode";
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.is_contiguous() && on_boundary(out, 16), op,
              ": out must be a contiguous 2-D CUDA tensor [N][K] on a 16-byte boundary");
  const auto type = out.scalar_type();
  const int kind = type == torch::kBFloat16 ? 1 : type == torch::kFloat16 ? 2 : type == torch::kFloat8_e4m3fn ? 3 : 0;
  TORCH_CHECK(kind != 0, op, ": out must be BF16, FP16 or FP8 E4M3, got ", type);
  const int64_t n = out.size(0), k = out.size(1);
  TORCH_CHECK(n >= 1 && k >= 16 && k % 16 == 0, op, ": out must be [N][K] with K a multiple of 16, got [", n, "][", k,
              "]");
  TORCH_CHECK(codes.is_cuda() && codes.dim() == 2 && codes.is_contiguous() && codes.scalar_type() == torch::kUInt8 &&
                  codes.size(0) == n && codes.size(1) * 2 == k && on_boundary(codes, 16),
              op, ": codes must be contiguous uint8 [N][K / 2] on a 16-byte boundary");
  TORCH_CHECK(scales.is_cuda() && scales.is_contiguous() && scales.element_size() == 1 && scales.dim() == 2 &&
                  scales.size(0) == n && scales.size(1) * 16 == k,
              op, ": scales must be contiguous E4M3 bytes [N][K / 16]");
  TORCH_CHECK(factor.is_cuda() && factor.is_contiguous() && factor.scalar_type() == torch::kFloat32 &&
                  factor.numel() == n && on_boundary(factor, 4),
              op, ": the per-row factor must be contiguous FP32 [N]");
  require_same_device(out, {&codes, &scales, &factor}, op);
  const c10::cuda::CUDAGuard guard(out.device());
  require_success(dg_enqueue_dequantize(codes.data_ptr<std::uint8_t>(),
                                        static_cast<const std::uint8_t*>(scales.data_ptr()), factor.data_ptr<float>(),
                                        out.data_ptr(), kind, static_cast<int>(n), static_cast<int>(k),
                                        at::cuda::getCurrentCUDAStream().stream()),
                  op);
}

int64_t hardware_decode(const torch::Tensor& device_of) {
  TORCH_CHECK(device_of.is_cuda(), "hardware_decode: the tensor names a CUDA device");
  const c10::cuda::CUDAGuard guard(device_of.device());
  const int answer = dg_hardware_decode();
  TORCH_CHECK(answer >= 0, "hardware_decode: ", device_of.device(), " cannot run this library (built for sm_100a only)");
  return answer;
}

// Any number of BF16 rows (the quantizers serve prompts as well as decode steps).
void require_rows_to_quantize(const torch::Tensor& x, const char* op) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16 && x.size(0) >= 1, op,
              ": x must be a 2-D BF16 CUDA tensor [rows][K] with at least one row");
  TORCH_CHECK(x.stride(1) == 1 && x.stride(0) % 8 == 0 && on_boundary(x, 16), op,
              ": rows of x must be contiguous and start on 16-byte boundaries");
}

void quantize_fp8_rows(const torch::Tensor& x, torch::Tensor& q, torch::Tensor& scale) {
  const char* op = "quantize_fp8_rows";
  require_rows_to_quantize(x, op);
  const int64_t rows = x.size(0), k = x.size(1);
  TORCH_CHECK(q.is_cuda() && q.dim() == 2 && q.element_size() == 1 && q.size(0) == rows && q.size(1) == k &&
                  q.stride(1) == 1,
              op, ": q must hold one byte per value, [rows][K] with contiguous rows");
  TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == torch::kFloat32 && scale.is_contiguous() &&
                  scale.numel() == rows,
              op, ": scale must be contiguous FP32 [rows]");
  require_same_device(x, {&q, &scale}, op);
  const c10::cuda::CUDAGuard guard(x.device());
  require_success(dg_enqueue_quantize_fp8_rows(x.data_ptr(), x.stride(0), static_cast<int>(rows), static_cast<int>(k),
                                               static_cast<std::uint8_t*>(q.data_ptr()), q.stride(0),
                                               scale.data_ptr<float>(), at::cuda::getCurrentCUDAStream().stream()),
                  op);
}

void quantize_nvfp4(const torch::Tensor& x, double input_scale, torch::Tensor& codes, torch::Tensor& scales) {
  const char* op = "quantize_nvfp4";
  require_rows_to_quantize(x, op);
  const int64_t rows = x.size(0), k = x.size(1);
  TORCH_CHECK(k >= 16 && k % 16 == 0, op, ": K must be a multiple of 16, got ", k);
  TORCH_CHECK(input_scale > 0, op, ": the input scale must be positive");
  TORCH_CHECK(codes.is_cuda() && codes.element_size() == 1 && codes.is_contiguous() &&
                  codes.numel() == rows * (k / 2) && on_boundary(codes, 8),
              op, ": codes must be contiguous bytes [rows][K / 2] on an 8-byte boundary");
  const int64_t tiled = ((rows + 127) / 128) * 128 * (((k / 16) + 3) / 4) * 4;
  TORCH_CHECK(scales.is_cuda() && scales.element_size() == 1 && scales.is_contiguous() && scales.numel() == tiled, op,
              ": scales must be ", tiled, " bytes: [rows][K / 16] in 128 x 4 tiles, rows padded to 128 and blocks to 4");
  require_same_device(x, {&codes, &scales}, op);
  const float g = static_cast<float>(input_scale);
  const c10::cuda::CUDAGuard guard(x.device());
  require_success(dg_enqueue_quantize_nvfp4(x.data_ptr(), x.stride(0), static_cast<int>(rows), static_cast<int>(k), g,
                                            1.0f / g, static_cast<std::uint8_t*>(codes.data_ptr()),
                                            static_cast<std::uint8_t*>(scales.data_ptr()),
                                            at::cuda::getCurrentCUDAStream().stream()),
                  op);
}

TORCH_LIBRARY(DG_TORCH_NAMESPACE, ops) {
  ops.def("gemv(Tensor x, Tensor codes, Tensor scales, Tensor inverse, bool blocked, Tensor! out) -> ()");
  ops.def("gemv_fp8(Tensor x, Tensor codes, Tensor scales, Tensor! out) -> ()");
  ops.def("gemv_bf16(Tensor x, Tensor w, Tensor! out) -> ()");
  ops.def("hardware_decode(Tensor device_of) -> int");
  ops.def("decode(Tensor codes, Tensor scales, Tensor factor, Tensor! out) -> ()");
  // the activation quantizers of the reference's mma-rows package, same schemas (mma-rows/torch-ext/torch_binding.cpp:11-12)
  ops.def("quantize_fp8_rows(Tensor x, Tensor! q, Tensor! scale) -> ()");
  ops.def("quantize_nvfp4(Tensor x, float input_scale, Tensor! codes, Tensor! scales) -> ()");
}

TORCH_LIBRARY_IMPL(DG_TORCH_NAMESPACE, CUDA, ops) {
  ops.impl("gemv", &gemv);
  ops.impl("gemv_fp8", &gemv_fp8);
  ops.impl("gemv_bf16", &gemv_bf16);
  ops.impl("hardware_decode", &hardware_decode);
  ops.impl("decode", &decode);
  ops.impl("quantize_fp8_rows", &quantize_fp8_rows);
  ops.impl("quantize_nvfp4", &quantize_nvfp4);
}
