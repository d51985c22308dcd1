// TEST INFRASTRUCTURE ONLY. C-ABI shim over the reference's own raw CUDA API, so that the unmodified reference kernel
// (decode-gemv/decode_gemv_cuda/decode_gemv.cu, compiled from where it lies in the reference checkout) can be run
// beside the product on a GPU box: as a second opinion on parity and as the GPU comparator in the bench. Nothing
// shipped links or loads this.
#include "decode_gemv.h"   // the reference's header, found through -I <reference>/decode-gemv/decode_gemv_cuda

namespace ref = crit::kernels::decode_gemv;

extern "C" {

__attribute__((visibility("default"))) int ref_enqueue_nvfp4(const void* x, int ldx, int x_is_bf16,
                                                            const unsigned char* codes, const unsigned char* scales,
                                                            int blocked, const float* inverse, void* out, int ldo,
                                                            int out_kind, int M, int N, int K, void* stream) {
  return (int)ref::enqueue_gemv(x, ldx, x_is_bf16 != 0, codes, scales, blocked != 0, inverse, out, ldo, out_kind == 0,
                                M, N, K, static_cast<cudaStream_t>(stream));
}

__attribute__((visibility("default"))) int ref_enqueue_fp8(const void* x, int ldx, int x_is_bf16,
                                                          const unsigned char* codes, const float* row_scale,
                                                          const unsigned char* mx_scale, void* out, int ldo,
                                                          int out_kind, int M, int N, int K, void* stream) {
  return (int)ref::enqueue_gemv_fp8(x, ldx, x_is_bf16 != 0, codes, row_scale, mx_scale, out, ldo, out_kind == 0, M, N,
                                    K, static_cast<cudaStream_t>(stream));
}

__attribute__((visibility("default"))) int ref_enqueue_bf16(const void* x, int ldx, const void* w, void* out, int ldo,
                                                           int out_kind, int M, int N, int K, void* stream) {
  return (int)ref::enqueue_gemv_bf16(x, ldx, w, out, ldo, out_kind == 0, M, N, K, static_cast<cudaStream_t>(stream));
}

__attribute__((visibility("default"))) int ref_hardware_decode(void) { return ref::hardware_decode(); }

}  // extern "C"
