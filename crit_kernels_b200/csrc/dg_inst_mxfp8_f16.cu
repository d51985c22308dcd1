// Kernels for M = 1..16: format FMT_MXFP8, activations __half.
#include "dg_inst.cuh"
DG_TABLE(dg_table_mxfp8_f16, dg::FMT_MXFP8, __half)
