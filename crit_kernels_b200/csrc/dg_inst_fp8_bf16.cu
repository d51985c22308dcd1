// Kernels for M = 1..16: format FMT_FP8, activations __nv_bfloat16.
#include "dg_inst.cuh"
DG_TABLE(dg_table_fp8_bf16, dg::FMT_FP8, __nv_bfloat16)
