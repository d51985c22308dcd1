// Batched kernels (several GEMVs a launch) for M = 1..16: format FMT_NVFP4, activations __nv_bfloat16.
#include "dg_inst.cuh"
DG_BATCH_TABLE(dg_batch_table_nvfp4_bf16, dg::FMT_NVFP4, __nv_bfloat16)
