// Kernels for M = 1..16: format FMT_FP8, activations __half.
#include "dg_inst.cuh"
DG_TABLE(dg_table_fp8_f16, dg::FMT_FP8, __half)
