// SwiGLU between the gate_up and down projections: out[row][k] = silu(gate_up[row][k]) * gate_up[row][inter + k], FP32
// arithmetic as the reference declares it (dg_swiglu.cuh; int-block-experts/int_block_cuda/int_block.cu:275-282 and its
// entry point :326-331), inputs and outputs FP32 or BF16 (one rounding to BF16 where the output is the next GEMV's
// activations). One thread eight values where rows are 16-byte aligned, else one. The NVFP4 GEMV can also form these
// activations itself while it stages them (dg_enqueue_nvfp4_swiglu), which this kernel serves as the unfused form of.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/decode_gemv_b200.h"
#include "dg_swiglu.cuh"

namespace {

template <bool IN_F32, bool OUT_F32>
__global__ void __launch_bounds__(256) swiglu_kernel(const void* __restrict__ gate_up, long long ldg, int rows, int inter,
                                                     void* __restrict__ out, long long ldo, int vector) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int per_row = vector ? inter >> 3 : inter;
  const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= (long long)rows * per_row) return;
  const int row = (int)(id / per_row), c = (int)(id - (long long)row * per_row);
  auto load = [&](size_t at) -> float {
    return IN_F32 ? reinterpret_cast<const float*>(gate_up)[at]
                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(gate_up)[at]);
  };
  auto store = [&](size_t at, float v) {
    if (OUT_F32) reinterpret_cast<float*>(out)[at] = v;
    else reinterpret_cast<__nv_bfloat16*>(out)[at] = __float2bfloat16_rn(v);
  };
  const size_t in0 = (size_t)row * ldg, out0 = (size_t)row * ldo;
  if (!vector) {
    store(out0 + c, dg::swiglu_value(load(in0 + c), load(in0 + inter + c)));
    return;
  }
  const int k = c << 3;
  float v[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = dg::swiglu_value(load(in0 + k + j), load(in0 + inter + k + j));
#pragma unroll
  for (int j = 0; j < 8; ++j) store(out0 + k + j, v[j]);   // consecutive: the compiler forms the vector accesses
}

bool aligned(const void* p, uintptr_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }

}  // namespace

extern "C" int dg_enqueue_swiglu(const void* gate_up, long long ldg, int in_is_f32, int rows, int inter, void* out,
                                 long long ldo, int out_is_f32, void* stream) {
  if (!gate_up || !out || rows < 0 || inter < 0 || ldg < 2LL * inter || ldo < inter) return (int)cudaErrorInvalidValue;
  if ((long long)rows * inter == 0) return (int)cudaSuccess;
  const int in_size = in_is_f32 ? 4 : 2, out_size = out_is_f32 ? 4 : 2;
  if (!aligned(gate_up, in_size) || !aligned(out, out_size)) return (int)cudaErrorInvalidValue;
  const int vector = inter % 8 == 0 && ldg % 8 == 0 && ldo % 8 == 0 && aligned(gate_up, 16) && aligned(out, 16);
  const long long threads = (long long)rows * (vector ? inter / 8 : inter);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)((threads + 255) / 256));
  config.blockDim = dim3(256);
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  cudaError_t e;
  if (in_is_f32 && out_is_f32) e = cudaLaunchKernelEx(&config, swiglu_kernel<true, true>, gate_up, ldg, rows, inter, out, ldo, vector);
  else if (in_is_f32) e = cudaLaunchKernelEx(&config, swiglu_kernel<true, false>, gate_up, ldg, rows, inter, out, ldo, vector);
  else if (out_is_f32) e = cudaLaunchKernelEx(&config, swiglu_kernel<false, true>, gate_up, ldg, rows, inter, out, ldo, vector);
  else e = cudaLaunchKernelEx(&config, swiglu_kernel<false, false>, gate_up, ldg, rows, inter, out, ldo, vector);
  return (int)(e != cudaSuccess ? e : cudaGetLastError());
}
