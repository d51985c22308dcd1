// Activation quantizers for B200 (sm_100a): BF16 rows to FP8 E4M3 with one scale per row, and to NVFP4 (E2M1 codes,
// one E4M3 scale per 16 values, scales in cuBLASLt's 128 x 4 tiled layout). The step just before a W8A8 / W4A4
// projection; they replace the reference's quantize_fp8_rows and quantize_nvfp4 (mma-rows/mma_rows_cuda/
// mma_rows.cu:15-140 kernels, :320-340 entry points; arithmetic in tile_parts.cuh:23-64, :301-331) bit for bit:
//
//   FP8 rows   scale = max(amax * fp32(1 / 448), 1e-12); q = E4M3(clamp(x / scale, +-448)), IEEE division, round to
//              nearest even. A NaN in a row makes its scale NaN (torch's amax).
//   NVFP4      per 16 values: s = E4M3(min((amax * fp32(1 / 6)) * g, 448)); d = max(e4m3(s) * (1 / g), 1e-30);
//              code = E2M1(x / d), nearest with ties to the even code, magnitudes above 6 to 6, the sign bit set for
//              every negative quotient, all codes 0 where e4m3(s) is not > 0.
//
// Machine mapping (not the reference's): a row of the FP8 quantizer is read from HBM once: one bulk copy (TMA, 1-D)
// brings it into shared memory, the CTA takes the maximum and quantizes from there, 16 output bytes per thread and
// store; rows that do not fit or are not 16-byte aligned are read twice through L2 instead. The NVFP4 quantizer gives a
// thread four consecutive blocks (128 input bytes, 32 code bytes, one 32-bit word of tiled scales) and converts with
// the hardware E2M1 / E4M3 conversions.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/decode_gemv_b200.h"

namespace {

constexpr float kRcp448 = 1.0f / 448.0f;   // a division by a constant is a product with its FP32 reciprocal in the
constexpr float kRcp6 = 1.0f / 6.0f;       // framework whose quantizers these reproduce
constexpr int kRowThreads = 256;
constexpr int kRowSmemLimit = 200 * 1024;
constexpr unsigned long long kCopyWaitNs = 2000000000ull;

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
// The larger of two values, NaN if either is (one instruction; BF16 pairs keep the maximum exactly).
__device__ __forceinline__ float nanmax(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ uint32_t amax2(uint32_t pair, uint32_t m) {   // per half: max(|pair|, m), NaN kept
  uint32_t r;
  asm("{\n\t.reg .b32 a;\n\tabs.bf16x2 a, %1;\n\tmax.NaN.bf16x2 %0, a, %2;\n\t}" : "=r"(r) : "r"(pair), "r"(m));
  return r;
}
__device__ __forceinline__ uint32_t amax8(const uint4& v, uint32_t m) {
  return amax2(v.w, amax2(v.z, amax2(v.y, amax2(v.x, m))));
}
__device__ __forceinline__ float amax_of(uint32_t m) { return nanmax(bf16_lo(m), bf16_hi(m)); }
// Two FP32 -> two E4M3 bytes (low byte = lo), round to nearest even, saturating.
__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float e4m3_value(uint32_t byte) {
  uint32_t h;
  asm("{\n\t.reg .b16 t;\n\tcvt.u16.u32 t, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, t;\n\t}" : "=r"(h) : "r"(byte & 0xffu));
  return __half2float(__ushort_as_half((unsigned short)(h & 0xffffu)));
}
// The clamp to +-448 that the quantizer's definition names is the saturating conversion's: every quotient beyond
// 448 (at most by a rounding of the scale) converts to 448 either way, NaN to NaN.
//
// x / d, correctly rounded, for many x over one d whose quotients stay within FP32's normal range (SAFE): with
// r = RN(1 / d) computed once, q0 = RN(x r), the exact residual e = x - d q0 (one FMA) and q = RN(q0 + e r) give the
// IEEE quotient: the tail of the usual division sequence without its per-element reciprocal refinement. A zero
// quotient keeps its own sign where that matters (KEEP_ZERO: the correction would turn -0 into +0). Quotients too
// small for an exact residual convert to zero whatever their last bits are. Otherwise the full division runs.
template <bool SAFE, bool KEEP_ZERO>
__device__ __forceinline__ float quotient(float x, float d, float r) {
  if constexpr (!SAFE) return __fdiv_rn(x, d);
  const float q0 = __fmul_rn(x, r);
  const float q1 = __fmaf_rn(__fmaf_rn(-d, q0, x), r, q0);
  return KEEP_ZERO && q0 == 0.f ? q0 : q1;
}
template <bool SAFE>
__device__ __forceinline__ uint32_t fp8_quad(uint32_t w0, uint32_t w1, float d, float r) {
  return e4m3x2(quotient<SAFE, true>(bf16_lo(w0), d, r), quotient<SAFE, true>(bf16_hi(w0), d, r)) |
         (e4m3x2(quotient<SAFE, true>(bf16_lo(w1), d, r), quotient<SAFE, true>(bf16_hi(w1), d, r)) << 16);
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The second pass over a row: 16 (or 8) values a thread and store where the output allows it.
template <bool SAFE>
__device__ __forceinline__ void quantize_row(const __nv_bfloat16* xr, const uint4* row_smem, uint8_t* qr, int K, float d,
                                             int staged, bool aligned_in, int vector_out, int tid) {
  const float r = SAFE ? __frcp_rn(d) : 0.f;
  if (aligned_in) {
    const uint4* rv = staged ? row_smem : reinterpret_cast<const uint4*>(xr);
    if (vector_out && (K & 15) == 0) {   // 16 values -> one 16-byte store
      for (int i = tid; i < (K >> 4); i += kRowThreads) {
        const uint4 a = staged ? rv[2 * i] : __ldg(rv + 2 * i), b = staged ? rv[2 * i + 1] : __ldg(rv + 2 * i + 1);
        reinterpret_cast<uint4*>(qr)[i] = make_uint4(fp8_quad<SAFE>(a.x, a.y, d, r), fp8_quad<SAFE>(a.z, a.w, d, r),
                                                     fp8_quad<SAFE>(b.x, b.y, d, r), fp8_quad<SAFE>(b.z, b.w, d, r));
      }
    } else if (vector_out) {             // 8 values -> one 8-byte store
      for (int i = tid; i < (K >> 3); i += kRowThreads) {
        const uint4 a = staged ? rv[i] : __ldg(rv + i);
        reinterpret_cast<uint2*>(qr)[i] = make_uint2(fp8_quad<SAFE>(a.x, a.y, d, r), fp8_quad<SAFE>(a.z, a.w, d, r));
      }
    } else {
      for (int i = tid; i < (K >> 3); i += kRowThreads) {
        const uint4 a = staged ? rv[i] : __ldg(rv + i);
        const uint32_t lo = fp8_quad<SAFE>(a.x, a.y, d, r), hi = fp8_quad<SAFE>(a.z, a.w, d, r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          qr[8 * i + j] = (uint8_t)(lo >> (8 * j));
          qr[8 * i + 4 + j] = (uint8_t)(hi >> (8 * j));
        }
      }
    }
  } else {
    for (int k = tid; k < K; k += kRowThreads)
      qr[k] = (uint8_t)(e4m3x2(quotient<SAFE, true>(__bfloat162float(xr[k]), d, r), 0.f) & 0xffu);
  }
}

// One CTA a row. `staged`: the row (K a multiple of 8, 16-byte aligned, within shared memory) arrives by one bulk copy.
__global__ void __launch_bounds__(kRowThreads) fp8_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int K,
                                                               uint8_t* __restrict__ q, long long ldq,
                                                               float* __restrict__ scale, int staged, int vector_out) {
  extern __shared__ __align__(128) unsigned char row_smem[];
  __shared__ __align__(8) unsigned long long bar;
  __shared__ float part[kRowThreads / 32];
  __shared__ float row_scale;
  __shared__ int failed;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const __nv_bfloat16* xr = x + (size_t)row * ldx;
  uint8_t* qr = q + (size_t)row * ldq;
  const uint32_t bar_addr = (uint32_t)__cvta_generic_to_shared(&bar);
  if (tid == 0) {
    failed = 0;
    if (staged) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_addr) : "memory");
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");   // x is the previous kernel's output
  float m = 0.f;
  uint32_t m2 = 0u;   // running maximum of BF16 pairs
  if (staged) {
    if (tid == 0) {
      const uint32_t bytes = (uint32_t)K * 2u;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       (uint32_t)__cvta_generic_to_shared(row_smem)),
                   "l"(xr), "r"(bytes), "r"(bar_addr)
                   : "memory");
    }
    // bounded wait for the copy (it cannot fail on valid arguments; the bound keeps a bad pointer from hanging)
    const unsigned long long start = global_ns();
    uint32_t ok = 0;
    for (uint32_t i = 1; !ok; ++i) {
      asm volatile(
          "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(bar_addr)
          : "memory");
      if (!ok && (i & 255u) == 0u && (failed || global_ns() - start > kCopyWaitNs)) {
        failed = 1;
        break;
      }
    }
    if (!ok) return;
    const uint4* rv = reinterpret_cast<const uint4*>(row_smem);
    for (int i = tid; i < (K >> 3); i += kRowThreads) m2 = amax8(rv[i], m2);
    m = amax_of(m2);
  } else if ((K & 7) == 0 && (ldx & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const uint4* rv = reinterpret_cast<const uint4*>(xr);
    for (int i = tid; i < (K >> 3); i += kRowThreads) m2 = amax8(__ldg(rv + i), m2);
    m = amax_of(m2);
  } else {
    for (int k = tid; k < K; k += kRowThreads) m = nanmax(m, fabsf(__bfloat162float(xr[k])));
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) m = nanmax(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) part[warp] = m;
  __syncthreads();
  if (tid == 0) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < kRowThreads / 32; ++w) a = nanmax(a, part[w]);
    const float sc = a * kRcp448;
    row_scale = sc < 1e-12f ? 1e-12f : sc;
    scale[row] = row_scale;
  }
  __syncthreads();
  const float sc = row_scale;
  const bool aligned_in = staged || ((K & 7) == 0 && (ldx & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0);
  // a finite scale bounds every quotient of the row by 448 (1 + a rounding): the short division; NaN or infinite
  // rows take the full one
  if (sc <= 1e30f)
    quantize_row<true>(xr, reinterpret_cast<const uint4*>(row_smem), qr, K, sc, staged, aligned_in, vector_out, tid);
  else
    quantize_row<false>(xr, reinterpret_cast<const uint4*>(row_smem), qr, K, sc, staged, aligned_in, vector_out, tid);
}

// Byte offset of block j of row n in cuBLASLt's 128 x 4 tiled scale layout with ct tiles per tile row.
__device__ __forceinline__ size_t tiled_offset(int n, int j, int ct) {
  const int r = n & 127;
  return ((size_t)(n >> 7) * ct + (j >> 2)) * 512 + (size_t)(r & 31) * 16 + (r >> 5) * 4 + (j & 3);
}

// Two quotients -> two E2M1 codes in one byte (low nibble = lo). v + 0 turns a negative zero into +0 (code 0, as a
// comparison with zero sees it); every other negative quotient keeps its sign bit, also when it rounds to zero.
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
  uint16_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}"
      : "=h"(r)
      : "f"(hi + 0.0f), "f"(lo + 0.0f));
  return r;
}

// 16 values (8 BF16 pairs) -> scale byte (returned) and 8 code bytes (lo, hi).
__device__ __forceinline__ uint32_t nvfp4_block(const uint4& v0, const uint4& v1, float g, float g_rcp, uint32_t& lo,
                                                uint32_t& hi) {
  const float amax = amax_of(amax8(v1, amax8(v0, 0u)));
  float bs = (amax * kRcp6) * g;
  bs = bs > 448.f ? 448.f : bs;
  const uint32_t sbits = e4m3x2(bs, 0.f) & 0xffu;
  float d = e4m3_value(sbits) * g_rcp;
  const bool zero = !(d > 0.f);
  d = d < 1e-30f ? 1e-30f : d;
  const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  lo = hi = 0u;
  if (zero) return sbits;
  // a block whose quotients cannot leave FP32's range takes the short division (a zero quotient's sign is dropped by
  // the conversion's + 0 anyway); the rest (values near FP32's limits) the full one
  if (amax < 1e8f) {
    const float r = __frcp_rn(d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = e2m1x2(quotient<true, false>(bf16_lo(w[i]), d, r), quotient<true, false>(bf16_hi(w[i]), d, r));
      if (i < 4) lo |= byte << (8 * i);
      else hi |= byte << (8 * (i - 4));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = e2m1x2(__fdiv_rn(bf16_lo(w[i]), d), __fdiv_rn(bf16_hi(w[i]), d));
      if (i < 4) lo |= byte << (8 * i);
      else hi |= byte << (8 * (i - 4));
    }
  }
  return sbits;
}

// One thread four consecutive blocks (one 32-bit word of the tiled scales) of the padded grid
// [rows_padded][blocks_padded / 4].
__global__ void __launch_bounds__(256) nvfp4_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, int M, int K,
                                                    float g, float g_rcp, uint8_t* __restrict__ codes,
                                                    uint8_t* __restrict__ scales, int rows_padded, int quads) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= (long long)rows_padded * quads) return;
  const int row = (int)(id / quads), quad = (int)(id - (long long)row * quads);
  uint32_t word = 0;
  const int blocks = K >> 4;
  if (row < M) {
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * ldx + 64 * quad);
    uint4 v[8];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const bool in = 4 * quad + b < blocks;
      v[2 * b] = in ? __ldg(src + 2 * b) : make_uint4(0u, 0u, 0u, 0u);
      v[2 * b + 1] = in ? __ldg(src + 2 * b + 1) : make_uint4(0u, 0u, 0u, 0u);
    }
    uint2* dst = reinterpret_cast<uint2*>(codes + (size_t)row * (K >> 1) + 32 * quad);
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      if (4 * quad + b < blocks) {
        uint32_t lo, hi;
        word |= nvfp4_block(v[2 * b], v[2 * b + 1], g, g_rcp, lo, hi) << (8 * b);
        dst[b] = make_uint2(lo, hi);
      }
    }
  }
  *reinterpret_cast<uint32_t*>(scales + tiled_offset(row, 4 * quad, quads)) = word;
}

bool aligned(const void* p, uintptr_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }

template <typename... Args>
cudaError_t launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&config, kernel, args...);
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

extern "C" {

int dg_enqueue_quantize_fp8_rows(const void* x, long long ldx, int M, int K, uint8_t* q, long long ldq, float* scale,
                                 void* stream) {
  if (M < 1 || K < 1 || !x || !q || !scale || ldx < K || ldq < K || !aligned(x, 2) || !aligned(scale, 4))
    return (int)cudaErrorInvalidValue;
  const size_t row_bytes = (size_t)K * 2;
  const int staged = K % 8 == 0 && ldx % 8 == 0 && aligned(x, 16) && row_bytes <= (size_t)kRowSmemLimit;
  const int vector_out = K % 16 == 0 ? (ldq % 16 == 0 && aligned(q, 16)) : (ldq % 8 == 0 && aligned(q, 8));
  const size_t smem = staged ? row_bytes : 0;
  if (smem > 48 * 1024) {
    // opt in above the default limit; per device, not a stream operation (costs nothing after the first call)
    static thread_local int opted[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!opted[dev]) {
      const cudaError_t e =
          cudaFuncSetAttribute(fp8_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRowSmemLimit);
      if (e != cudaSuccess) return (int)e;
      opted[dev] = 1;
    }
  }
  return (int)launch_pdl(fp8_rows_kernel, dim3((unsigned)M), dim3(kRowThreads), smem, static_cast<cudaStream_t>(stream),
                         static_cast<const __nv_bfloat16*>(x), ldx, K, q, ldq, scale, staged, vector_out);
}

int dg_enqueue_quantize_nvfp4(const void* x, long long ldx, int M, int K, float input_scale, float input_rcp,
                              uint8_t* codes, uint8_t* blocked_scales, void* stream) {
  if (M < 1 || K < 16 || K % 16 || !x || !codes || !blocked_scales || ldx < K || ldx % 8 || !aligned(x, 16) ||
      !aligned(codes, 8) || !aligned(blocked_scales, 4) || !(input_scale > 0.f))
    return (int)cudaErrorInvalidValue;
  const int rows_padded = (M + 127) / 128 * 128, quads = (K / 16 + 3) / 4;
  const long long threads = (long long)rows_padded * quads;
  return (int)launch_pdl(nvfp4_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0,
                         static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x), ldx, M, K, input_scale,
                         input_rcp, codes, blocked_scales, rows_padded, quads);
}

}  // extern "C"
