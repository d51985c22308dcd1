// Expands to the table of the sixteen kernels (M = 1..16) of one format and activation type.
#pragma once
#include "dg_kernel.cuh"
#include "dg_tables.h"

#define DG_K(FMT, M, XT) reinterpret_cast<const void*>(&dg::gemv_kernel<FMT, M, XT>)
#define DG_TABLE(NAME, FMT, XT)                                                                                     \
  const void* const NAME[16] = {DG_K(FMT, 1, XT),  DG_K(FMT, 2, XT),  DG_K(FMT, 3, XT),  DG_K(FMT, 4, XT),          \
                                DG_K(FMT, 5, XT),  DG_K(FMT, 6, XT),  DG_K(FMT, 7, XT),  DG_K(FMT, 8, XT),          \
                                DG_K(FMT, 9, XT),  DG_K(FMT, 10, XT), DG_K(FMT, 11, XT), DG_K(FMT, 12, XT),         \
                                DG_K(FMT, 13, XT), DG_K(FMT, 14, XT), DG_K(FMT, 15, XT), DG_K(FMT, 16, XT)};

#define DG_KB(FMT, M, XT) reinterpret_cast<const void*>(&dg::gemv_batch_kernel<FMT, M, XT>)
#define DG_BATCH_TABLE(NAME, FMT, XT)                                                                               \
  const void* const NAME[16] = {DG_KB(FMT, 1, XT),  DG_KB(FMT, 2, XT),  DG_KB(FMT, 3, XT),  DG_KB(FMT, 4, XT),      \
                                DG_KB(FMT, 5, XT),  DG_KB(FMT, 6, XT),  DG_KB(FMT, 7, XT),  DG_KB(FMT, 8, XT),      \
                                DG_KB(FMT, 9, XT),  DG_KB(FMT, 10, XT), DG_KB(FMT, 11, XT), DG_KB(FMT, 12, XT),     \
                                DG_KB(FMT, 13, XT), DG_KB(FMT, 14, XT), DG_KB(FMT, 15, XT), DG_KB(FMT, 16, XT)};
