// TEST INFRASTRUCTURE ONLY. C-ABI shim over the reference's SwiGLU (int-block-experts/int_block_cuda/int_block.h:
// enqueue_swiglu), so that the unmodified reference kernel, compiled from where it lies in the reference checkout, can
// be run beside the product on a GPU box as the bit-exact checker. Nothing shipped links or loads this.
#include "int_block.h"   // the reference's header, found through -I <reference>/int-block-experts/int_block_cuda

extern "C" __attribute__((visibility("default"))) int ref_swiglu(const float* gate_up, int inter, int rows, float* out,
                                                                 void* stream) {
  return (int)crit::techniques::int_block::enqueue_swiglu(gate_up, inter, rows, out, static_cast<cudaStream_t>(stream));
}
