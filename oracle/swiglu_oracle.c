/* TEST INFRASTRUCTURE ONLY: CPU restatement of the reference's SwiGLU (int-block-experts/int_block_cuda/
 * int_block.cu:55-69 exp_declared, :275-282 swiglu_kernel), the checker of crit_kernels_b200/csrc/dg_swiglu.cu(h).
 * Every step is one IEEE single-precision operation (fmaf is the fused multiply-add of the C library, rintf rounds to
 * nearest even), in the reference's order, so the results are its bits. Built by oracle/build_oracle.py with
 * gcc -O2 -ffp-contract=off into oracle/_ref/libswiglu_oracle.so; nothing shipped links or loads it.
 * Pinned on a GPU box against the reference's own kernel (oracle/_ref/libint_block_ref.so, tests/test_swiglu_gpu.py). */
#include <math.h>
#include <stdint.h>
#include <string.h>

static float exp_declared(float x) {
  x = x > 88.0f ? 88.0f : x < -87.0f ? -87.0f : x;
  const float n = rintf(x * 1.44269504f);
  float r = fmaf(n, -0.693145752f, x);
  r = fmaf(n, -1.42860677e-06f, r);
  float p = 1.98412698e-04f;
  p = fmaf(p, r, 1.38888889e-03f);
  p = fmaf(p, r, 8.33333333e-03f);
  p = fmaf(p, r, 4.16666667e-02f);
  p = fmaf(p, r, 1.66666667e-01f);
  p = fmaf(p, r, 0.5f);
  p = fmaf(p, r, 1.0f);
  p = fmaf(p, r, 1.0f);
  const int32_t bits = ((int32_t)n + 127) << 23;
  float scale;
  memcpy(&scale, &bits, 4);
  return p * scale;
}

/* out[row][k] = silu(gate_up[row][k]) * gate_up[row][inter + k], rows of gate_up 2 * inter apart, FP32. */
void swiglu_f32(const float* gate_up, int inter, int rows, float* out) {
  for (int row = 0; row < rows; ++row)
    for (int k = 0; k < inter; ++k) {
      const float gate = gate_up[(size_t)row * 2 * inter + k], up = gate_up[(size_t)row * 2 * inter + inter + k];
      const float silu = gate / (1.0f + exp_declared(-gate));
      out[(size_t)row * inter + k] = silu * up;
    }
}
