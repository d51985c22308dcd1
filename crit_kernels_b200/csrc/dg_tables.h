// Kernel tables: one entry per activation-row count 1..16, defined by the instantiation units (dg_inst_*.cu) and
// read by the dispatcher (dg_abi.cu).
#pragma once

extern const void* const dg_table_bf16[16];
extern const void* const dg_table_fp8_bf16[16];
extern const void* const dg_table_fp8_f16[16];
extern const void* const dg_table_mxfp8_bf16[16];
extern const void* const dg_table_mxfp8_f16[16];
extern const void* const dg_table_nvfp4_bf16[16];
extern const void* const dg_table_nvfp4_f16[16];
extern const void* const dg_batch_table_nvfp4_bf16[16];   // gemv_batch_kernel, NVFP4, BF16 activations
