// NVFP4 dequantizers for B200 (sm_100a): the matrix's values [N][K] as BF16 / FP16, or as FP8 E4M3 in units of a
// per-row factor. The "dequantize" half of the reference's dequantize-then-matmul path.
//
// Replaces the Triton kernels of the reference package decode-gemv (torch-ext/decode_gemv/triton_gemv.py:156-176
// `_decode_kernel` / `decode`, :179-200 `_decode_fp8_kernel` / `decode_fp8`). Contract, as the reference's test pins
// it (tests/test_decode_gemv.py:131-140): value = e2m1(code) * scale (exact in FP32) times the row's factor, one FP32
// product, rounded once to the output type; the FP8 form clamps to +-448 before rounding to nearest even.
//
// Pure streaming, HBM-bound and write-dominated: per value 0.5 B of codes + 1/16 B of scales in, 2 B (or 1 B) out.
// A lane writes one 16-byte vector per step: 8 values from one 32-bit word of codes for the 16-bit types, 16 values
// (one scale block) from two words for FP8, so a warp reads 128 (256) consecutive bytes and writes 512 consecutive
// bytes per step; four steps are loaded before any is converted.
// Rows are dealt to blockIdx.y, a row's words to blockIdx.x; the grid is a multiple of the SM count.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "../../include/decode_gemv_b200.h"
#include "dg_kernel.cuh"

namespace {

enum : int { DQ_BF16 = 1, DQ_F16 = 2, DQ_E4M3 = 3 };
constexpr int kThreads = 256;
constexpr int kBatch = 4;   // 16-byte output units a thread has in flight

__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

__device__ __forceinline__ void unpack2(dg::pk2 a, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a.v));
}

// 8 codes (word c, element 2i in the low nibble of byte i) -> 8 FP32 values: (e2m1 * scale) * factor.
__device__ __forceinline__ void values8(uint32_t c, float scale, float factor, float (&v)[8]) {
  dg::pk2 w[4];
  dg::decode_e2m1(c, w);                                   // (element 2q, element 2q + 1) of byte q
  const dg::pk2 s2 = dg::pack2(scale, scale), f2 = dg::pack2(factor, factor);
#pragma unroll
  for (int q = 0; q < 4; ++q) unpack2(dg::fmul2(dg::fmul2(w[q], s2), f2), v[2 * q], v[2 * q + 1]);
}

template <int OUT>
__device__ __forceinline__ uint32_t round2(float lo, float hi) {   // two values of a 16-bit type in one word
  if constexpr (OUT == DQ_BF16) {
    const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&t);
  } else {
    const __half2 t = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&t);
  }
}
// Four values as E4M3 bytes; the saturating conversion gives +-448 beyond +-448, as the reference's clamp before its
// rounding.
__device__ __forceinline__ uint32_t round4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// A lane's unit is 16 output bytes: one word of codes (8 values) for the 16-bit types, two words (16 values, one
// scale block) for FP8. `unit` counts such units from the start of the matrix.
template <int OUT> struct Unit { static constexpr int WORDS = OUT == DQ_E4M3 ? 2 : 1; };

template <int OUT>
__global__ void __launch_bounds__(kThreads)
    dequantize_kernel(const uint32_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                      const float* __restrict__ factor, uint4* __restrict__ out, int N, int K) {
  constexpr int WORDS = Unit<OUT>::WORDS;
  const int units = K / (8 * WORDS);                        // per row
  const int stride = gridDim.x * kThreads;
  for (int row = blockIdx.y; row < N; row += gridDim.y) {
    const float f = __ldg(factor + row);
    const uint32_t* crow = codes + (size_t)row * (K / 8);
    const uint8_t* srow = scales + (size_t)row * (K / 16);
    uint4* orow = out + (size_t)row * units;
    for (int u0 = blockIdx.x * kThreads + threadIdx.x; u0 < units; u0 += kBatch * stride) {
      uint32_t c[kBatch][WORDS] = {}, sb[kBatch] = {};
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int u = u0 + b * stride;
        if (u < units) {
          if constexpr (WORDS == 2) {
            const uint2 two = __ldg(reinterpret_cast<const uint2*>(crow) + u);
            c[b][0] = two.x;
            c[b][1] = two.y;
            sb[b] = __ldg(srow + u);                        // the unit is one scale block
          } else {
            c[b][0] = __ldg(crow + u);
            sb[b] = __ldg(srow + (u >> 1));                 // one scale per 16 values = per two words
          }
        }
      }
#pragma unroll
      for (int b = 0; b < kBatch; ++b) {
        const int u = u0 + b * stride;
        if (u < units) {
          const float scale = e4m3_to_f32(sb[b]);
          float v[8];
          uint4 o;
          values8(c[b][0], scale, f, v);
          if constexpr (WORDS == 2) {
            o.x = round4_e4m3(v[0], v[1], v[2], v[3]);
            o.y = round4_e4m3(v[4], v[5], v[6], v[7]);
            values8(c[b][1], scale, f, v);
            o.z = round4_e4m3(v[0], v[1], v[2], v[3]);
            o.w = round4_e4m3(v[4], v[5], v[6], v[7]);
          } else {
            o.x = round2<OUT>(v[0], v[1]);
            o.y = round2<OUT>(v[2], v[3]);
            o.z = round2<OUT>(v[4], v[5]);
            o.w = round2<OUT>(v[6], v[7]);
          }
          orow[u] = o;
        }
      }
    }
  }
}

// SM count of the current device (0: not a device this library runs on), looked up once per device.
int sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  int sms = cache[dev].load(std::memory_order_relaxed);
  if (sms == 0) {
    int major = 0, count = 0;
    const bool ok = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess &&
                    major == 10 &&
                    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && count > 0;
    sms = ok ? count : -1;
    cache[dev].store(sms, std::memory_order_relaxed);
  }
  return sms > 0 ? sms : 0;
}

bool aligned(const void* ptr, uintptr_t bytes) { return reinterpret_cast<uintptr_t>(ptr) % bytes == 0; }

}  // namespace

extern "C" DG_API int dg_enqueue_dequantize(const uint8_t* codes, const uint8_t* scales, const float* factor, void* out,
                                     int out_kind, int N, int K, void* stream) {
  if (N < 1 || K < 16 || K % 16 || out_kind < DQ_BF16 || out_kind > DQ_E4M3) return (int)cudaErrorInvalidValue;
  if (!codes || !scales || !factor || !out || !aligned(codes, 16) || !aligned(out, 16) || !aligned(factor, 4))
    return (int)cudaErrorInvalidValue;
  const int sms = sm_count();
  if (sms < 1) return (int)cudaErrorInvalidDevice;
  const int units = K / (out_kind == DQ_E4M3 ? 16 : 8);      // 16-byte output vectors per row
  int gx = (units + kThreads * kBatch - 1) / (kThreads * kBatch);
  if (gx > 8) gx = 8;
  int gy = (sms * 8 + gx - 1) / gx;                          // about eight CTAs per SM in all
  if (gy > N) gy = N;
  if (gy > 65535) gy = 65535;
  const dim3 grid(gx, gy), block(kThreads);
  const uint32_t* c32 = reinterpret_cast<const uint32_t*>(codes);
  uint4* o = static_cast<uint4*>(out);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out_kind == DQ_BF16) dequantize_kernel<DQ_BF16><<<grid, block, 0, s>>>(c32, scales, factor, o, N, K);
  else if (out_kind == DQ_F16) dequantize_kernel<DQ_F16><<<grid, block, 0, s>>>(c32, scales, factor, o, N, K);
  else dequantize_kernel<DQ_E4M3><<<grid, block, 0, s>>>(c32, scales, factor, o, N, K);
  return (int)cudaGetLastError();
}
