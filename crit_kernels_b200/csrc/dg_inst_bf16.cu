// Kernels for M = 1..16: format FMT_BF16, activations __nv_bfloat16.
#include "dg_inst.cuh"
DG_TABLE(dg_table_bf16, dg::FMT_BF16, __nv_bfloat16)
