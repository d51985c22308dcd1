// Kernels for M = 1..16: format FMT_NVFP4, activations __half.
#include "dg_inst.cuh"
DG_TABLE(dg_table_nvfp4_f16, dg::FMT_NVFP4, __half)
