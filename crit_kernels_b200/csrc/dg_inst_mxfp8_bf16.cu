// Kernels for M = 1..16: format FMT_MXFP8, activations __nv_bfloat16.
#include "dg_inst.cuh"
DG_TABLE(dg_table_mxfp8_bf16, dg::FMT_MXFP8, __nv_bfloat16)
