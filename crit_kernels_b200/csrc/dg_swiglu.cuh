// SwiGLU of one (gate, up) pair in FP32, in the reference's declared arithmetic (int-block-experts/int_block_cuda/
// int_block.cu:55-69 exp_declared, :275-282 swiglu_kernel): every operation is a named IEEE operation, so that a CPU
// with fmaf reproduces the bits. silu(g) = g / (1 + exp(-g)); exp by range reduction with n = rint(x * log2(e)),
// r = x - n ln 2 in two FMAs, a degree-7 polynomial, and 2^n built in the exponent field.
#pragma once
#include <cuda_runtime.h>

namespace dg {

__device__ __forceinline__ float exp_declared(float x) {
  x = x > 88.0f ? 88.0f : x < -87.0f ? -87.0f : x;
  const float n = rintf(__fmul_rn(x, 1.44269504f));
  float r = __fmaf_rn(n, -0.693145752f, x);
  r = __fmaf_rn(n, -1.42860677e-06f, r);
  float p = 1.98412698e-04f;
  p = __fmaf_rn(p, r, 1.38888889e-03f);
  p = __fmaf_rn(p, r, 8.33333333e-03f);
  p = __fmaf_rn(p, r, 4.16666667e-02f);
  p = __fmaf_rn(p, r, 1.66666667e-01f);
  p = __fmaf_rn(p, r, 0.5f);
  p = __fmaf_rn(p, r, 1.0f);
  p = __fmaf_rn(p, r, 1.0f);
  return __fmul_rn(p, __int_as_float(((int)n + 127) << 23));
}

__device__ __forceinline__ float swiglu_value(float gate, float up) {
  const float silu = __fdiv_rn(gate, __fadd_rn(1.0f, exp_declared(-gate)));
  return __fmul_rn(silu, up);
}

}  // namespace dg
