// TEST INFRASTRUCTURE ONLY. C-ABI shim over the reference's activation quantizers (mma-rows/mma_rows_cuda/mma_rows.h:
// enqueue_quantize_fp8_rows, enqueue_quantize_nvfp4), so that the unmodified reference kernels, compiled from where
// they lie in the reference checkout, can be run beside the product on a GPU box as the bit-exact checker. Nothing
// shipped links or loads this.
#include "mma_rows.h"   // the reference's header, found through -I <reference>/mma-rows/mma_rows_cuda

namespace ref = crit::kernels::mma_rows;

extern "C" {

__attribute__((visibility("default"))) int ref_quantize_fp8_rows(const void* x, long long ldx, int M, int K,
                                                                unsigned char* q, long long ldq, float* scale,
                                                                void* stream) {
  return (int)ref::enqueue_quantize_fp8_rows(x, ldx, M, K, q, ldq, scale, static_cast<cudaStream_t>(stream));
}

__attribute__((visibility("default"))) int ref_quantize_nvfp4(const void* x, long long ldx, int M, int K,
                                                             float input_scale, float input_rcp, unsigned char* codes,
                                                             unsigned char* blocked_scales, void* stream) {
  return (int)ref::enqueue_quantize_nvfp4(x, ldx, M, K, input_scale, input_rcp, codes, blocked_scales,
                                          static_cast<cudaStream_t>(stream));
}

}  // extern "C"
