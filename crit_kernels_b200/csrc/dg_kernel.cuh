// Weight-only decode GEMV for B200 (sm_100a): out[m][n] = scale[n] * sum_k x[m][k] * w[n][k] for 1..16 activation
// rows, weights stored as BF16, FP8 E4M3 (row scale), MXFP8 (E8M0 per 32) or NVFP4 (E2M1 codes, E4M3 per 16).
//
// Replaces the kernels of the reference package decode-gemv (decode_gemv_cuda/decode_gemv.cu:85 gemv_kernel,
// :191 bf16_kernel, :285 fp8_kernel). Same formats, same contract (FP32 sums whose order never depends on the row
// count), a different machine mapping:
//
//   * one persistent CTA per SM: C consumer warps + P producer warps (12 + 4 down to 8 + 0, by format and M). The matrix
//     rows are split into one contiguous range per CTA; a range is walked in tiles of C*r rows (r rows per consumer
//     warp) and each tile in K windows.
//   * the producer warps stream every window of a tile into a shared-memory ring: one cp.async.bulk (TMA 1-D bulk
//     copy, mbarrier complete_tx) per weight row (and per row of block scales), issued by the producers' lanes in
//     parallel, plus the matching window of the activations as 16-byte cp.async copies into a bank-swizzled layout.
//     Bytes in flight are set by the ring (up to ~200 KB per SM), not by registers. Where the arithmetic, not HBM,
//     is the limit (larger M) the CTA has no producer warp: its consumer warps issue the same copies between stages.
//   * consumer warp w owns rows w, w+C, ... of the tile. Lane l owns the 16-byte blocks l, l+32, ... of each row and
//     keeps two FP32 chains per (row, m): even and odd elements, advanced together by one packed fma.rn.f32x2 or, where
//     the arithmetic is the limit, by two mixed-precision fma.rn.f32.bf16 / .f16 (same bits: the products are exact).
//     The chains visit the blocks in ascending order, the two chains are added, and one xor-shuffle tree (16, 8, 4, 2,
//     1) adds the lanes; the row scale multiplies once and the result is rounded once to the output type.
//
// A row's summation order is therefore a function of K and the format alone: it does not depend on M, on the rows a
// warp holds, on the tile or window sizes the launch picked, on the CTA count, or on which slice of the matrix a
// device holds. Every product is exact in FP32 (weights and block scales have few significant bits), NVFP4 block
// scales multiply a 16-element partial sum (one fma per block and row instead of one multiply per weight).
#pragma once

#include <cuda.h>   // CUtensorMap (type only; the driver entry point is looked up at run time)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <type_traits>

#include "dg_swiglu.cuh"

namespace dg {

enum : int { FMT_BF16 = 0, FMT_FP8 = 1, FMT_MXFP8 = 2, FMT_NVFP4 = 3 };
enum : int { SCALES_NONE = 0, SCALES_STAGED = 1, SCALES_DIRECT = 2, SCALES_BLOCKED = 3 };
enum : int { OUT_F32 = 0, OUT_BF16 = 1, OUT_F16 = 2 };

constexpr int kMaxStages = 12;
constexpr int RMAX_ALL = 4;                // most rows a consumer warp holds in any kernel
constexpr int kMeetBytes = 16 * RMAX_ALL * 16 * 4;   // SwiGLU epilogue: 16 warps x (4 rows x 16 activation rows) FP32
constexpr int kStepBytes = 512;            // 32 lanes x 16 bytes of one weight row
constexpr int kSmemHeader = 256;           // mbarriers + abort flag
constexpr int kSmemLimit = 232448;         // 227 KB of dynamic shared memory per CTA on sm_100
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // bounded waits give up after this (default; the host
                                                             // can set another limit, Params::wait_limit_ns)

// status word bits written on a wait that ran out (never expected; the host can read the word)
constexpr int kStatusProducerTimeout = 1;
constexpr int kStatusConsumerTimeout = 2;
constexpr int kStatusGatherTimeout = 4;
constexpr int kMaxRanks = 8;
// Time stamps (%globaltimer, ns) a CTA leaves in Params::trace when a trace buffer is set: kernel entry, the wait for
// the previous kernel of the stream passed, first stage full, last stage consumed, last warp done; then the SM id.
constexpr int kTraceSlots = 8;
enum : int { TRACE_ENTRY = 0, TRACE_DEP = 1, TRACE_FIRST_FULL = 2, TRACE_LAST_CONSUMED = 3, TRACE_EXIT = 4, TRACE_SM = 5 };

template <int FMT> struct Format;
template <> struct Format<FMT_BF16>  { static constexpr int E = 8,  SCB = 0;  };   // elements / scale bytes per
template <> struct Format<FMT_FP8>   { static constexpr int E = 16, SCB = 0;  };   // 16-byte block and per 512-byte
template <> struct Format<FMT_MXFP8> { static constexpr int E = 16, SCB = 16; };   // step of one row
template <> struct Format<FMT_NVFP4> { static constexpr int E = 32, SCB = 64; };

// CTA shape per (format, M): a speed choice, never a row's bits. Register need decides it: the accumulators take
// 2 * rows * M registers and the held operand (activations or decoded weights) 8-16 per activation row or weight row.
//   class 0   M small: the kernel is HBM-bound. 12 consumer + 4 producer warps (14 + 2 where two_producers says so;
//             128 registers each): as many warps
//             as the register file gives, to hide shared-memory and conversion latencies; every SM sub-partition
//             hosts the same number of consumers.
//   class 1   M medium: 11 consumer + 1 producer warps, or 12 consumer warps that issue the copies themselves
//             (168 registers each).
//   class 2   M large: the kernel is FP32-FMA-bound. No producer warp; 8 to 16 consumer warps by (format, M), see
//             class2_warps / class2_rows.
//             In classes 1 and 2 the consumers' instruction issue is the limit and a sub-partition's time is that of
//             the consumers it hosts, so the consumers should be spread evenly: one producer warp keeps up with the
//             copies and leaves one sub-partition a consumer short (measured against 10 + 2 and 6 + 2 warps: 4-8 %
//             and 10-17 % faster); no producer warp at all leaves none short but adds the copies to the consumers'
//             instruction streams (measured against 11 + 1 and 7 + 1: class 2 up to 14 % faster, never slower;
//             class 1 4-8 % faster for BF16 and MXFP8, 3-6 % slower for FP8 and NVFP4, which keep the producer).
//             Moving the class limits either way measured 15-30 % slower.
// Classes 0 and 1 hold the converted activations of a block and stream the rows past them; class 2 holds the rows'
// decoded weights and streams the activation rows.
// One warp issues a 1-D bulk copy only every ~60 clocks, so full groups of rows travel as one 2-D tensor copy and
// only a tile's ragged remainder as per-row copies.
__host__ __device__ constexpr int shape_class(int fmt, int m) {
  return fmt == FMT_NVFP4 ? (m <= 2 ? 0 : m <= 4 ? 1 : 2) : (m <= 4 ? 0 : m <= 8 ? 1 : 2);
}
// CTAs that share an SM (each with its share of the shared memory; the grid is this many per SM). BF16 class 0 runs
// two CTAs of 7 + 1 warps: the next kernel's CTA moves in and starts its copies as soon as the first of the two
// leaves (3-7 % faster over back-to-back calls at 8192 x 8192 than one CTA of 14 + 2; the other formats measured
// 10-20 % slower as two CTAs of 6 + 2 than as one of 12 + 4).
__host__ __device__ constexpr int ctas_per_sm(int fmt, int m) { return fmt == FMT_BF16 && shape_class(fmt, m) == 0 ? 2 : 1; }
__host__ __device__ constexpr bool few_rows(int fmt, int m) { return shape_class(fmt, m) < 2; }
// (BF16 weights, the lightest arithmetic per byte, measured 13-19 % faster with 14 + 2 warps per SM than with 12 + 4;
// they run as two CTAs of 7 + 1, see ctas_per_sm.)
// class 1 of the formats with the lighter arithmetic per byte (BF16, MXFP8) and class 2 of all: no producer warp.
__host__ __device__ constexpr bool self_fed(int fmt, int m) {
  return shape_class(fmt, m) == 2 || (shape_class(fmt, m) == 1 && (fmt == FMT_BF16 || fmt == FMT_MXFP8));
}
// Class 2 by (format, M), measured on 28672 x 8192 (16384 x 8192 for BF16) over the candidates 8 warps x 4 rows,
// 12 x 3, 12 x 4 and 16 x 2 (255, 168, 168 and 128 registers per thread): up to 14 % between them. NVFP4 also on
// 8192 x 8192, 8192 x 28672 and 57344 x 8192: at M = 8 the 16 x 2 shape is 2 % ahead of 8 x 4 on the large matrices
// and 20-23 % on the two with 8192 rows (55 rows per CTA).
// Class 0 with 14 + 2 warps instead of 12 + 4: FP8 and NVFP4 at M <= 2 measured 1.5-2 % faster at 28672 x 8192 and
// NVFP4 7 % faster at 8192 x 8192 (M = 1); MXFP8 measured 10 % slower at M = 2 and stays.
__host__ __device__ constexpr bool two_producers(int fmt, int m) { return (fmt == FMT_FP8 || fmt == FMT_NVFP4) && m <= 2; }
__host__ __device__ constexpr int class2_warps(int fmt, int m) {
  return fmt == FMT_FP8 ? (m <= 13 ? 12 : 8)
         : fmt == FMT_BF16 ? (m <= 14 ? 12 : 8)
         : fmt == FMT_NVFP4 ? (m == 8 || m >= 11 ? 16 : 12) : 8;
}
__host__ __device__ constexpr int class2_rows(int fmt, int m) {
  return fmt == FMT_NVFP4 ? (m == 5 ? 4 : m == 8 || m >= 11 ? 2 : 3) : fmt == FMT_BF16 && m >= 12 && m <= 14 ? 3 : 4;
}
__host__ __device__ constexpr int consumer_warps(int fmt, int m) {
  return shape_class(fmt, m) == 0 ? (fmt == FMT_BF16 ? 7 : two_producers(fmt, m) ? 14 : 12)
         : shape_class(fmt, m) == 1 ? (self_fed(fmt, m) ? 12 : 11) : class2_warps(fmt, m);
}
__host__ __device__ constexpr int producer_warps(int fmt, int m) {
  return shape_class(fmt, m) == 0 ? (fmt == FMT_BF16 ? 1 : two_producers(fmt, m) ? 2 : 4) : self_fed(fmt, m) ? 0 : 1;
}
// Kernels that advance their chains with the mixed-precision FMA instead of the packed FP32 FMA (same bits; see f2):
// where the arithmetic is the limit, one issue slot per product without any conversion of the activations beats
// half a slot per product plus the conversions. MXFP8 stays on the FP32 path: its weights carry their block scale,
// and weight x 2^(e - 127) is not always a BF16 value.
__host__ __device__ constexpr bool use_mixed(int fmt, int m) {
  return fmt != FMT_MXFP8 && (shape_class(fmt, m) == 2 || (shape_class(fmt, m) == 1 && fmt != FMT_FP8) ||
                              (fmt == FMT_BF16 && m <= 2));   // BF16 weights need no conversion at all: M FMAs per
                                                              // weight against 1 + M / 2 instructions packed
}
// Rows a consumer warp holds at once (register budget).
__host__ __device__ constexpr int rows_max(int fmt, int m) {
  return shape_class(fmt, m) == 2 ? class2_rows(fmt, m) : 4;
}
// Resident activations (Params::x_resident, decided by the launch plan): class 0 of FP8 / NVFP4, where the whole
// [M][K] activations are small, keeps them in shared memory behind the ring for the whole kernel instead of copying a
// window of them into every ring stage: the consumer warps fetch them once, while the first weights are on their way.
// (also NVFP4's class 1, M = 3 and 4: a mixed-FMA kernel whose FP16 steps spare it the weights' conversion to BF16)
__host__ __device__ constexpr bool resident_capable(int fmt, int m) {
  return ((fmt == FMT_FP8 || fmt == FMT_NVFP4) && shape_class(fmt, m) == 0) ||
         (fmt == FMT_NVFP4 && shape_class(fmt, m) == 1);
}
constexpr int kResidentLimit = 96 * 1024;   // bytes of activations (and their flags) a kernel keeps resident at most
// How a kernel instance advances its chains, by the activations' type too.
//   MIXED     the mixed-precision FMA throughout: use_mixed, and every FP16-activation kernel of the formats whose
//             decoded weights are FP16 values already (E4M3, E2M1): nothing is converted at all.
//   HALF_RES  BF16 activations of a resident_capable kernel: when the activations are resident, each 512-byte step
//             of them (64 * E elements of every activation row) is kept as FP16 if every value of it is an FP16
//             value too (|x| <= 65504, and FP16 carries BF16's 8 significant bits down to 2^-17), and the consumers
//             run the FP16 mixed-FMA body on that step: about 2 instead of 3.5 instructions per weight at M = 1. A
//             step with any other value (tiny, huge, infinite, NaN) stays BF16 and takes the kernel's other body
//             (packed FP32, or the BF16 mixed FMA with converted weights). Every product is exact either way and the
//             additions are the same, so are the bits.
template <int FMT, int M, typename XT>
struct Arithmetic {
  static constexpr bool HALF_X = std::is_same<XT, __half>::value;
  static constexpr bool MIXED = use_mixed(FMT, M) || (HALF_X && (FMT == FMT_FP8 || FMT == FMT_NVFP4));
  static constexpr bool HALF_RES = !HALF_X && resident_capable(FMT, M);
};

struct Params {
  const void* x;             // [M][ldx] BF16 or FP16
  const uint8_t* w;          // weight rows, row_bytes apart
  const uint8_t* scales;     // NVFP4 E4M3 [N][K/16] (or tiled), MXFP8 E8M0 [N][K/32]; else null
  const float* row_scale;    // FP8 row scale / NVFP4 inverse global scale [N]; else null
  void* out;                 // [M][ldo]
  int* status;               // device word for kStatus* bits
  int ldx, ldo, out_kind;
  int N, K;
  int row_bytes;             // bytes of one weight row
  int nblk;                  // 16-byte blocks per row
  int scale_row_bytes;       // bytes of one row-major scale row
  int scale_mode;            // SCALES_*
  int ct;                    // tiled scales: 4-block tiles per tile row
  int steps;                 // 512-byte steps per ring stage
  int stages;                // ring depth
  int rows_per_warp;         // r: a full tile is (consumer warps) * r rows
  int stage_bytes;           // bytes of one ring stage
  int use_2d;                // 1: tmap_w (and tmap_sc when scales are staged) are valid
  int early_weights;         // 1: weight copies may be issued before the previous kernel of the stream completed
  int split_tail;            // 1: a short last tile and the tile before it are walked as two equal tiles (see Walk)
  // SwiGLU epilogue (pairs > 0): the matrix is a gate_up projection of 2 * pairs rows, gate rows [0, pairs) and up rows
  // [pairs, 2 pairs); N counts the rows as the tiles walk them (see Walk). A warp holds row k of both halves side by
  // side and writes out[m][k] = silu(gate) * up (FP32, one rounding) instead of the two sums: `pairs` columns.
  int pairs;
  // Resident activations (resident_capable kernels; 0 = the activations travel through the ring stages): the
  // kernel's dynamic shared memory holds, x_res_off bytes in, ceil(nblk / 32) steps of [M][64 * E elements] laid out
  // as in a stage, then one flag byte per step (1 = the step is held as FP16, see Arithmetic::HALF_RES).
  int x_resident, x_res_off;
  unsigned long long* trace; // diagnostic (dg_set_trace): kTraceSlots time stamps per CTA, or null
  unsigned long long wait_limit_ns;   // every wait in the kernel gives up after this long (status word, then leaves)
  // All-gather epilogue (world >= 1, 0 = off): this rank's [M][N] results go into slot `rank` of its own
  // [world][M][N] buffer; every CTA then copies its rows to the same slot of every other rank's buffer (peer_out[q],
  // peer-mapped addresses) and counts itself done in word 2 of this rank's counter block; the last CTA adds 1 to
  // word `gather_slot` (0 or 1) of every rank's block (peer_flag[q]) and waits until its own word holds `world`, then
  // clears it: when the kernel ends, every rank's data has landed here.
  int world, rank, gather_slot, gather_nowait;   // nowait: signal only; dg_enqueue_gather_wait collects later
  void* peer_out[kMaxRanks];
  unsigned int* peer_flag[kMaxRanks];
  // Tensor maps over the weight rows and the row-major scale rows as 8-byte elements: box = (consumer warps) rows
  // x one window. Rows are 16-byte multiples apart, which the encoder requires.
  alignas(64) CUtensorMap tmap_w;
  alignas(64) CUtensorMap tmap_sc;
};

// ---------------------------------------------------------------------------------------------------------------
// PTX wrappers: mbarrier, 1-D bulk copy (TMA), 16-byte cp.async tied to an mbarrier.

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory loads by 32-bit shared-space address: the ring is addressed with one base register per stage plus
// constants, instead of 64-bit generic pointer arithmetic per load. Volatile keeps them after the barrier waits.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts_u8(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ldg_nc128(const void* ptr) {   // memory nobody writes while the kernel runs
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}

// Two FP32 values in one 64-bit register pair, the operand form of the packed fma.rn.f32x2 / mul.rn.f32x2. Operands
// are packed once where they are produced and accumulators stay packed across the whole K loop, so that no
// pack / unpack moves surround the FMAs (measured: almost one extra instruction per packed FMA otherwise).
struct pk2 { unsigned long long v; };
__device__ __forceinline__ pk2 pack2(float lo, float hi) {
  pk2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ pk2 pack2_bits(uint32_t lo, uint32_t hi) {
  pk2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ float sum2(pk2 a) {   // low + high
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a.v));
  return lo + hi;
}
__device__ __forceinline__ pk2 ffma2(pk2 a, pk2 b, pk2 c) {   // (a.lo * b.lo + c.lo, a.hi * b.hi + c.hi), each IEEE RN
  pk2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d.v) : "l"(a.v), "l"(b.v), "l"(c.v));
  return d;
}
__device__ __forceinline__ pk2 fmul2(pk2 a, pk2 b) {
  pk2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d.v) : "l"(a.v), "l"(b.v));
  return d;
}
// The same two chains as two plain FP32 registers, for the kernels that advance them with the mixed-precision FMA
// (16-bit operands, FP32 addend and result, one rounding: fma.rn.f32.bf16 / fma.rn.f32.f16). The product of two 16-bit
// operands is exact in FP32, so the result is bit for bit that of the FP32 FMA on the converted operands; what the
// mixed form saves is the conversion of the activations to FP32, which it reads as loaded. There is no packed mixed
// form, so these kernels issue one FMA per product.
struct f2 { float lo, hi; };
__device__ __forceinline__ float sum2(f2 a) { return a.lo + a.hi; }
template <typename XT> struct Mixed;
template <> struct Mixed<__nv_bfloat16> {
  // (w.lo * x.lo + acc.lo, w.hi * x.hi + acc.hi): two BF16 pairs in 32-bit registers
  __device__ __forceinline__ static f2 fma2(uint32_t w, uint32_t x, f2 acc) {
    asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %2;\n\tmov.b32 {xl, xh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, wl, xl, %0;\n\tfma.rn.f32.bf16 %1, wh, xh, %1;\n\t}"
        : "+f"(acc.lo), "+f"(acc.hi) : "r"(w), "r"(x));
    return acc;
  }
  // Two FP16 values that are exact in BF16 (decoded E4M3 / E2M1) as a BF16 pair: through FP32, every step exact.
  __device__ __forceinline__ static uint32_t weights(uint32_t h) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&h));
    const __nv_bfloat162 p = __floats2bfloat162_rn(t.x, t.y);
    return *reinterpret_cast<const uint32_t*>(&p);
  }
};
template <> struct Mixed<__half> {
  __device__ __forceinline__ static f2 fma2(uint32_t w, uint32_t x, f2 acc) {
    asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %2;\n\tmov.b32 {xl, xh}, %3;\n\t"
        "fma.rn.f32.f16 %0, wl, xl, %0;\n\tfma.rn.f32.f16 %1, wh, xh, %1;\n\t}"
        : "+f"(acc.lo), "+f"(acc.hi) : "r"(w), "r"(x));
    return acc;
  }
  __device__ __forceinline__ static uint32_t weights(uint32_t h) { return h; }   // decoded weights are FP16 already
};
template <typename XT>
__device__ __forceinline__ f2 mixed_fma4(const uint32_t (&w)[4], const uint4& x, f2 a) {
  a = Mixed<XT>::fma2(w[0], x.x, a);
  a = Mixed<XT>::fma2(w[1], x.y, a);
  a = Mixed<XT>::fma2(w[2], x.z, a);
  return Mixed<XT>::fma2(w[3], x.w, a);
}
template <typename XT, int R, int M>
__device__ __forceinline__ void mixed_rows(const uint32_t (&w)[R][4], const uint4& x, f2 (&acc)[R][M], int m) {
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r][m] = mixed_fma4<XT>(w[r], x, acc[r][m]);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. False when it gave up or another thread of the CTA already had: the caller leaves its loops.
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void trace_stamp(unsigned long long* trace, int slot) {   // the latest stamp of a slot wins
  if (trace) atomicMax(trace + (size_t)blockIdx.x * kTraceSlots + slot, global_ns());
}
// The limit sits in shared memory right after the abort flag (written once by the kernel's first thread).
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const unsigned long long start = global_ns();
  const unsigned long long limit = *reinterpret_cast<const volatile unsigned long long*>(abort_flag + 2);
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0u) {
      if (*abort_flag) return false;
      if (global_ns() - start > limit) break;
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// 2-D tiled tensor copy: box of the tensor map at element column x, row y.
__device__ __forceinline__ void tensor_g2s(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------------------------------------------------------
// Element conversions. All exact.

__device__ __forceinline__ pk2 half2_bits_to_f32(uint32_t h) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
  return pack2(f.x, f.y);
}
__device__ __forceinline__ pk2 pair_to_f32(uint32_t v, __nv_bfloat16) {   // two BF16 -> two FP32
  // byte permute for the low element: keeps the shift off the FMA pipe, which the packed FMAs need
  return pack2_bits(__byte_perm(v, 0u, 0x1044u), v & 0xffff0000u);
}
__device__ __forceinline__ pk2 pair_to_f32(uint32_t v, __half) {          // two FP16 -> two FP32
  return half2_bits_to_f32(v);
}
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t v) {                // low 16 bits: two E4M3 -> two FP32
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}
// E8M0 exponent byte as FP32 2^(e-127); e = 0 is the FP32 subnormal 2^-127 and e = 255 is NaN, as the reference
// decodes them (decode_gemv.cu:275-278).
__device__ __forceinline__ float e8m0_to_f32(uint32_t e) {
  return __uint_as_float(e == 0u ? 0x00400000u : e == 255u ? 0x7fc00000u : e << 23);
}
// Offset of the byte of 16-block j (j even) of row n in cuBLASLt's 128 x 4 tiled scale layout, ct tiles per tile
// row: the layout the reference reads at decode_gemv.cu:78-82.
__device__ __forceinline__ size_t tiled_scale_offset(int n, int j, int ct) {
  const int r = n & 127;
  return ((size_t)(n >> 7) * ct + (j >> 2)) * 512 + (size_t)(r & 31) * 16 + (r >> 5) * 4 + (j & 3);
}

__device__ __forceinline__ void store_out(void* out, int kind, size_t idx, float v) {
  if (kind == OUT_F32) reinterpret_cast<float*>(out)[idx] = v;
  else if (kind == OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(out)[idx] = __float2half_rn(v);
}

// ---------------------------------------------------------------------------------------------------------------
// Tile walk shared by producers and consumers: CTA c owns rows [lo, hi); tiles of CW * r rows, the last one shorter.

template <int CW>
struct Walk {
  int lo, hi, tile_rows, ntiles, nwin, win_bytes;
  int split_row0, split_first;   // split tail: first row and height of the last-but-one tile (split_first = 0: none)
  int pairs;                     // SwiGLU epilogue: rows per half of the gate_up matrix (0: an ordinary matrix)
  __device__ __forceinline__ Walk(const Params& p) {
    pairs = p.pairs;
    if (pairs) {
      // The tiles walk the rows in blocks of CW: block 2 b holds gate rows [b CW, (b + 1) CW), block 2 b + 1 the up
      // rows of the same columns, so that a warp's rows 2 j and 2 j + 1 of a tile are gate and up of one column. A CTA
      // owns whole pairs of blocks; [lo, hi) counts rows in that order (the last pair of blocks may be short).
      const int blocks = (pairs + CW - 1) / CW;
      lo = 2 * CW * (int)(((long long)blocks * blockIdx.x) / gridDim.x);
      hi = 2 * CW * (int)(((long long)blocks * (blockIdx.x + 1)) / gridDim.x);
    } else {
      lo = (int)(((long long)p.N * blockIdx.x) / gridDim.x);
      hi = (int)(((long long)p.N * (blockIdx.x + 1)) / gridDim.x);
    }
    tile_rows = CW * p.rows_per_warp;
    ntiles = (hi - lo + tile_rows - 1) / tile_rows;
    // A short last tile walks every K window for a few rows: with only `stages` windows in flight and almost no
    // bytes in each, it runs at DRAM latency, not bandwidth. For one activation row (the only case where it
    // measured faster: 8192 x 28672 NVFP4 45.5 -> 41.1 us) the last full tile and a remainder under a quarter of a
    // tile are therefore walked as two tiles of equal height (48 + 7 -> 28 + 27).
    split_first = 0;
    split_row0 = 0;
    const int rows = hi - lo, rem = rows % tile_rows;
    if (p.split_tail && !pairs && rows > tile_rows && rem > 0 && 4 * rem < tile_rows) {
      split_row0 = lo + (ntiles - 2) * tile_rows;
      split_first = (tile_rows + rem + 1) / 2;
    }
    win_bytes = p.steps * kStepBytes;
    nwin = (p.row_bytes + win_bytes - 1) / win_bytes;
  }
  // Group g of tile t (the rows a tile's consumer warps hold as their row g): first matrix row and row count (0..CW).
  __device__ __forceinline__ void group(int t, int g, int& row0, int& rows) const {
    if (pairs) {
      const int first = lo + t * tile_rows + g * CW;         // in walking order
      const int block = first / CW, k0 = (block >> 1) * CW;
      rows = first < hi ? max(0, min(CW, pairs - k0)) : 0;
      row0 = (block & 1) * pairs + k0;
    } else {
      int tile0, tile_n;
      tile(t, tile0, tile_n);
      row0 = tile0 + g * CW;
      rows = max(0, min(CW, tile_n - g * CW));
    }
  }
  // First row and height of tile t (ordinary matrices).
  __device__ __forceinline__ void tile(int t, int& row0, int& rows) const {
    if (split_first && t >= ntiles - 2) {
      row0 = t == ntiles - 2 ? split_row0 : split_row0 + split_first;
      rows = t == ntiles - 2 ? split_first : hi - row0;
    } else {
      row0 = lo + t * tile_rows;
      rows = min(tile_rows, hi - row0);
    }
  }
};

// Bytes of the scales of one group of `cw` rows in a stage, padded to the 128 bytes a tensor copy's destination
// must be aligned to.
__host__ __device__ constexpr int scale_group_bytes(int cw, int steps, int scb) { return (cw * steps * scb + 127) & ~127; }

// Shared-memory stage: [weights rows_cap x win_bytes][scales: r groups of CW rows x steps*SCB, each group padded to
// 128 bytes][x: steps x M x 64*E bytes, the activations of one 512-byte step of every activation row together]. Tile row t = w + CW * g is row w of group g.
template <int FMT, int M, int CW>
struct StageLayout {
  static constexpr int E = Format<FMT>::E, SCB = Format<FMT>::SCB;
  int w_row, sc_row, sc_group, sc_off, x_off;
  __device__ __forceinline__ StageLayout(const Params& p) {
    const int rows_cap = CW * p.rows_per_warp;
    w_row = p.steps * kStepBytes;
    sc_row = p.steps * SCB;
    sc_group = scale_group_bytes(CW, p.steps, SCB);
    sc_off = rows_cap * w_row;
    x_off = sc_off + p.rows_per_warp * sc_group;
  }
};

// 16-byte slot s of an activation row lands at slot s ^ ((s >> 3) & (NQ - 1)) (NQ = 16-byte slots a lane reads per
// block): the eight lanes of a quarter warp then read eight different bank groups.
template <int NQ>
__device__ __forceinline__ int swizzle_slot(int s) { return s ^ ((s >> 3) & (NQ - 1)); }

// ---------------------------------------------------------------------------------------------------------------
// Producer warps: `pl` is this thread's index among the 32 * PW producer lanes.

// Programmatic dependent launch: the next kernel of the stream may start while this one runs, and this one may have
// started while the previous one ran. `griddep_wait` returns once the previous kernel has completed and its writes
// are visible; without the launch attribute both are no-ops.
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <int FMT, int M, int CW, int PW>
struct Producer {
  static constexpr int E = Format<FMT>::E, SCB = Format<FMT>::SCB, NQ = E / 8, PL = 32 * PW;
  const Params& p;
  const Params& maps;   // where the tensor maps are read from: kernel parameter or global memory, never shared memory
                        // (p itself, unless p is a copy the CTA keeps in shared memory)
  const Walk<CW> wk;
  const StageLayout<FMT, M, CW> lay;
  const uint32_t ring, full0, empty0;
  const bool staged;
  const int pl;

  __device__ __forceinline__ Producer(const Params& p_, const Params& maps_, unsigned char* smem, uint32_t full0_,
                                      uint32_t empty0_, int pl_)
      : p(p_), maps(maps_), wk(p_), lay(p_), ring(smem_addr(smem) + kSmemHeader), full0(full0_), empty0(empty0_),
        staged(SCB != 0 && p_.scale_mode == SCALES_STAGED), pl(pl_) {}
  __device__ __forceinline__ Producer(const Params& p_, const Params& maps_, const Walk<CW>& wk_,
                                      const StageLayout<FMT, M, CW>& lay_, unsigned char* smem, uint32_t full0_,
                                      uint32_t empty0_, int pl_)
      : p(p_), maps(maps_), wk(wk_), lay(lay_), ring(smem_addr(smem) + kSmemHeader), full0(full0_), empty0(empty0_),
        staged(SCB != 0 && p_.scale_mode == SCALES_STAGED), pl(pl_) {}

  // Weight (and scale) copies of iteration `it` (tile it / nwin, window it % nwin) into stage s.
  // Full groups of CW rows travel as one 2-D tensor copy each (always the whole box: columns past the row's end are
  // zero-filled and still counted), the remainder as one 1-D bulk copy per row. One arrival carries the byte count
  // of them all; completions may land before it (the phase cannot end while this arrival and the producers'
  // cp.async arrivals are outstanding).
  __device__ __forceinline__ void weights(int it, int s) const {
    const int t = it / wk.nwin, win = it - t * wk.nwin;
    const uint32_t full = full0 + 8u * s;
    const uint32_t stage = ring + (uint32_t)s * p.stage_bytes;
    const int byte0 = win * wk.win_bytes;
    const int wbytes = min(wk.win_bytes, p.row_bytes - byte0);
    const int scbytes = staged ? (wbytes * SCB) >> 9 : 0;
    if (!wk.pairs) {
      // consecutive rows: the whole groups of CW rows as boxes, issued by as many lanes at once, the rest row by row
      int row0, rows;
      wk.tile(t, row0, rows);
      const int boxes = p.use_2d ? rows / CW : 0;
      const int box_rows = boxes * CW;
      if (pl == 0)
        mbar_arrive_expect_tx(full, (uint32_t)box_rows * (uint32_t)(lay.w_row + (staged ? lay.sc_row : 0)) +
                                        (uint32_t)(rows - box_rows) * (uint32_t)(wbytes + scbytes));
      if (pl < boxes) {
        tensor_g2s(stage + pl * CW * lay.w_row, &maps.tmap_w, byte0 >> 3, row0 + pl * CW, full);
        if (staged)
          tensor_g2s(stage + lay.sc_off + pl * lay.sc_group, &maps.tmap_sc, (win * lay.sc_row) >> 3, row0 + pl * CW, full);
      }
      for (int r = box_rows + pl; r < rows; r += PL) {
        const size_t n = (size_t)(row0 + r);
        bulk_g2s(stage + r * lay.w_row, p.w + n * p.row_bytes + byte0, (uint32_t)wbytes, full);
        if (staged)
          bulk_g2s(stage + lay.sc_off + (r / CW) * lay.sc_group + (r % CW) * lay.sc_row,
                   p.scales + n * p.scale_row_bytes + (size_t)win * lay.sc_row, (uint32_t)scbytes, full);
      }
      return;
    }
    // gate_up with the SwiGLU epilogue: groups of CW rows from the two halves in turn; a whole group is one box (one
    // lane each, issued together), a short one goes row by row
    uint32_t expect = 0;
    for (int g = 0; g < p.rows_per_warp; ++g) {
      int row0, rows;
      wk.group(t, g, row0, rows);
      expect += p.use_2d && rows == CW ? (uint32_t)CW * (uint32_t)(lay.w_row + (staged ? lay.sc_row : 0))
                                       : (uint32_t)rows * (uint32_t)(wbytes + scbytes);
    }
    if (pl == 0) mbar_arrive_expect_tx(full, expect);
    if (pl < p.rows_per_warp) {
      int row0, rows;
      wk.group(t, pl, row0, rows);
      if (p.use_2d && rows == CW) {
        tensor_g2s(stage + pl * CW * lay.w_row, &maps.tmap_w, byte0 >> 3, row0, full);
        if (staged)
          tensor_g2s(stage + lay.sc_off + pl * lay.sc_group, &maps.tmap_sc, (win * lay.sc_row) >> 3, row0, full);
      }
    }
    for (int g = 0; g < p.rows_per_warp; ++g) {
      int row0, rows;
      wk.group(t, g, row0, rows);
      if (rows == 0 || (p.use_2d && rows == CW)) continue;
      for (int r = pl; r < rows; r += PL) {
        const size_t n = (size_t)(row0 + r);
        bulk_g2s(stage + (g * CW + r) * lay.w_row, p.w + n * p.row_bytes + byte0, (uint32_t)wbytes, full);
        if (staged)
          bulk_g2s(stage + lay.sc_off + g * lay.sc_group + r * lay.sc_row,
                   p.scales + n * p.scale_row_bytes + (size_t)win * lay.sc_row, (uint32_t)scbytes, full);
      }
    }
  }

  // Activations of iteration `it`: wbytes / 16 blocks of E elements per row, 16 bytes (8 elements) per copy; then
  // this lane's arrival, which fires when its copies have landed.
  __device__ __forceinline__ void activations(int it, int s) const {
    if constexpr (resident_capable(FMT, M)) {
      if (p.x_resident) {   // nothing to copy: the lane's arrival alone
        cp_async_arrive_noinc(full0 + 8u * s);
        return;
      }
    }
    const int win = it % wk.nwin;
    const uint32_t full = full0 + 8u * s;
    const uint32_t stage = ring + (uint32_t)s * p.stage_bytes;
    const int byte0 = win * wk.win_bytes;
    const int wbytes = min(wk.win_bytes, p.row_bytes - byte0);
    const int slots = (wbytes >> 4) * NQ;
    const size_t xbyte0 = (size_t)(byte0 >> 4) * E * 2;
    const unsigned char* xg = reinterpret_cast<const unsigned char*>(p.x);
    constexpr int STEP_SLOTS = 32 * NQ;              // 16-byte slots of one step of one activation row (64 * E bytes)
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
      const uint32_t dst = stage + lay.x_off + m * (64 * E);
      const unsigned char* src = xg + (size_t)m * p.ldx * 2 + xbyte0;
      for (int sl = pl; sl < slots; sl += PL) {
        const int st = sl / STEP_SLOTS, in_step = sl - st * STEP_SLOTS;
        cp_async16(dst + st * (M * 64 * E) + swizzle_slot<NQ>(in_step) * 16, src + (size_t)sl * 16);
      }
    }
    cp_async_arrive_noinc(full);
  }

  // The same copies when all the CTA's threads share them (PL a multiple of a step's slots): a thread keeps one
  // slot position of every step and every (PL / slots-per-step)-th activation row, so its addresses advance by
  // constants.
  __device__ __forceinline__ void activations_shared(int it, int s) const {
    constexpr int STEP_SLOTS = 32 * NQ, MSTRIDE = PL / STEP_SLOTS;
    static_assert(PL % STEP_SLOTS == 0 && MSTRIDE >= 1, "copying threads must cover whole steps");
    const int win = it % wk.nwin;
    const int byte0 = win * wk.win_bytes;
    const int wbytes = min(wk.win_bytes, p.row_bytes - byte0);
    const int slots = (wbytes >> 4) * NQ;
    const int in_step = pl % STEP_SLOTS, m0 = pl / STEP_SLOTS;
    uint32_t dst = ring + (uint32_t)s * p.stage_bytes + lay.x_off + swizzle_slot<NQ>(in_step) * 16;
    const unsigned char* src =
        reinterpret_cast<const unsigned char*>(p.x) + (size_t)(byte0 >> 4) * E * 2 + (size_t)in_step * 16;
    const size_t xrow = (size_t)p.ldx * 2;
    for (int sl = in_step; sl < slots; sl += STEP_SLOTS, dst += M * 64 * E, src += STEP_SLOTS * 16) {
#pragma unroll
      for (int k = 0; k < (M + MSTRIDE - 1) / MSTRIDE; ++k) {
        const int m = m0 + k * MSTRIDE;
        if (m < M) cp_async16(dst + m * (64 * E), src + m * xrow);
      }
    }
    cp_async_arrive_noinc(full0 + 8u * s);
  }

  // One GEMV's iterations. The ring position (stage s, its phase parity) is the caller's and carries on from one
  // GEMV of a batch to the next; `first` is the kernel's first GEMV: only there the previous kernel of the stream may
  // still be running (wait before the activations; with static weights, after the first weight copies).
  __device__ __forceinline__ bool run(volatile int* abort_flag, int& s, uint32_t& parity, bool first) const {
    const int total = wk.ntiles * wk.nwin;
    int it = 0;
    if (first && p.early_weights) {
      // The weights do not depend on the previous kernel of the stream: fill the ring with them before waiting for
      // it; the activations (its output, typically) follow the wait. (First GEMV: the ring is empty, s = 0.)
      const int ahead = min(p.stages, total);
      for (int i = 0; i < ahead; ++i) weights(i, i);
      griddep_wait();
      for (int i = 0; i < ahead; ++i) activations(i, i);
      it = ahead;
      if (ahead == p.stages) parity ^= 1u;
      else s = ahead;
    } else if (first) {
      griddep_wait();
    }
    for (; it < total; ++it) {
      if (!mbar_wait(empty0 + 8u * s, parity ^ 1u, abort_flag)) {
        if ((pl & 31) == 0 && p.status) atomicOr(p.status, kStatusProducerTimeout);
        return false;
      }
      weights(it, s);
      activations(it, s);
      if (++s == p.stages) { s = 0; parity ^= 1u; }
    }
    return true;
  }
};

// ---------------------------------------------------------------------------------------------------------------
// Consumer bodies: one 16-byte block of each of R rows times M activation rows. `wrow` points at the block of the
// warp's first row in the stage, rows are `wstride` bytes apart; `xs` at the stage's activations.
// acc[r][m] = (even chain, odd chain). With few activation rows (FEW) the activations of the block are converted
// once and held while the rows stream past; otherwise the rows' weights are decoded once and held while the
// activation rows stream past. Per (row, m) both issue the same operations in the same order.

template <int NQ>
struct XOffsets {   // byte offsets of the lane's NQ swizzled slots inside one step of one activation row
  int off[NQ];
  __device__ __forceinline__ XOffsets(int lane) {
#pragma unroll
    for (int j = 0; j < NQ; ++j) off[j] = swizzle_slot<NQ>(lane * NQ + j) * 16;
  }
};

template <typename XT>
__device__ __forceinline__ void load_x8(uint32_t addr, pk2 (&x)[4]) {   // 8 activations -> 4 FP32 pairs
  const uint4 v = lds128(addr);
  x[0] = pair_to_f32(v.x, XT());
  x[1] = pair_to_f32(v.y, XT());
  x[2] = pair_to_f32(v.z, XT());
  x[3] = pair_to_f32(v.w, XT());
}
__device__ __forceinline__ pk2 fma4(const pk2 (&w)[4], const pk2 (&x)[4], pk2 a) {
  a = ffma2(w[0], x[0], a);
  a = ffma2(w[1], x[1], a);
  a = ffma2(w[2], x[2], a);
  return ffma2(w[3], x[3], a);
}

// 8 weights of a sub-block as 4 FP32 pairs.
__device__ __forceinline__ void decode_bf16(const uint4& v, pk2 (&w)[4]) {
  w[0] = pair_to_f32(v.x, __nv_bfloat16());
  w[1] = pair_to_f32(v.y, __nv_bfloat16());
  w[2] = pair_to_f32(v.z, __nv_bfloat16());
  w[3] = pair_to_f32(v.w, __nv_bfloat16());
}
// The conversions take their packed source from a 16-bit (E4M3 pair) or 8-bit (E2M1 pair) register; unpacking the
// word in PTX lets the assembler select the sub-word instead of shifting it out first.
__device__ __forceinline__ void decode_e4m3(uint32_t a, uint32_t b, pk2 (&w)[4]) {
  uint32_t h0, h1, h2, h3;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
      : "=r"(h0), "=r"(h1) : "r"(a));
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
      : "=r"(h2), "=r"(h3) : "r"(b));
  w[0] = half2_bits_to_f32(h0);
  w[1] = half2_bits_to_f32(h1);
  w[2] = half2_bits_to_f32(h2);
  w[3] = half2_bits_to_f32(h3);
}
__device__ __forceinline__ void decode_e2m1(uint32_t a, pk2 (&w)[4]) {
  uint32_t h0, h1, h2, h3;
  asm("{\n\t.reg .b8 c0, c1, c2, c3;\n\t"
      "mov.b32 {c0, c1, c2, c3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, c0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, c1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, c2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, c3;\n\t}"
      : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(a));
  w[0] = half2_bits_to_f32(h0);
  w[1] = half2_bits_to_f32(h1);
  w[2] = half2_bits_to_f32(h2);
  w[3] = half2_bits_to_f32(h3);
}

template <bool FEW, int M, int R, typename XT>
__device__ __forceinline__ void body_bf16(uint32_t wrow, const uint32_t (&woff)[R], uint32_t xs, pk2 (&acc)[R][M]) {
  constexpr int XROW = 64 * Format<FMT_BF16>::E;   // bytes between activation rows inside a step
  uint4 wv[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wv[r] = lds128(wrow + woff[r]);
  if constexpr (FEW) {
    pk2 xf[M][4];
#pragma unroll
    for (int m = 0; m < M; ++m) load_x8<XT>(xs + m * XROW, xf[m]);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      pk2 wf[4];
      decode_bf16(wv[r], wf);
#pragma unroll
      for (int m = 0; m < M; ++m) acc[r][m] = fma4(wf, xf[m], acc[r][m]);
    }
  } else {
    pk2 wf[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) decode_bf16(wv[r], wf[r]);
#pragma unroll
    for (int m = 0; m < M; ++m) {
      pk2 xf[4];
      load_x8<XT>(xs + m * XROW, xf);
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r][m] = fma4(wf[r], xf, acc[r][m]);
    }
  }
}

// FP8 / MXFP8: the block is two sub-blocks of 8 weights (words 0-1, words 2-3). `sc` holds the MXFP8 scale of each
// row's block (unused for FP8): every weight is multiplied by it (exact: a power of two).
template <bool FEW, bool MX, int M, int R, typename XT>
__device__ __forceinline__ void body_fp8(uint32_t wrow, const uint32_t (&woff)[R], const float (&sc)[R], uint32_t xs,
                                         const XOffsets<2>& xo, pk2 (&acc)[R][M]) {
  constexpr int XROW = 64 * Format<FMT_FP8>::E;   // bytes between activation rows inside a step
  uint4 wv[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wv[r] = lds128(wrow + woff[r]);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    if constexpr (FEW) {
      pk2 xf[M][4];
#pragma unroll
      for (int m = 0; m < M; ++m) load_x8<XT>(xs + m * XROW + xo.off[j], xf[m]);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        pk2 wf[4];
        decode_e4m3(j ? wv[r].z : wv[r].x, j ? wv[r].w : wv[r].y, wf);
        if (MX) {
          const pk2 s2 = pack2(sc[r], sc[r]);
#pragma unroll
          for (int q = 0; q < 4; ++q) wf[q] = fmul2(wf[q], s2);
        }
#pragma unroll
        for (int m = 0; m < M; ++m) acc[r][m] = fma4(wf, xf[m], acc[r][m]);
      }
    } else {
      pk2 wf[R][4];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        decode_e4m3(j ? wv[r].z : wv[r].x, j ? wv[r].w : wv[r].y, wf[r]);
        if (MX) {
          const pk2 s2 = pack2(sc[r], sc[r]);
#pragma unroll
          for (int q = 0; q < 4; ++q) wf[r][q] = fmul2(wf[r][q], s2);
        }
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        pk2 xf[4];
        load_x8<XT>(xs + m * XROW + xo.off[j], xf);
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r][m] = fma4(wf[r], xf, acc[r][m]);
      }
    }
  }
}

// NVFP4: the block is 32 codes = two scale blocks of 16 (words 0-1 with scale .x, words 2-3 with scale .y). The 16
// products of a scale block are summed first (two chains of 8, started by a multiply), then acc = fma(scale,
// partial, acc).
__device__ __forceinline__ pk2 dot16(const pk2 (&wa)[4], const pk2 (&wb)[4], const pk2 (&xa)[4],
                                     const pk2 (&xb)[4]) {
  pk2 part = fmul2(wa[0], xa[0]);
  part = ffma2(wa[1], xa[1], part);
  part = ffma2(wa[2], xa[2], part);
  part = ffma2(wa[3], xa[3], part);
  return fma4(wb, xb, part);
}

template <bool FEW, int M, int R, typename XT>
__device__ __forceinline__ void body_nvfp4(uint32_t wrow, const uint32_t (&woff)[R], const float2 (&sc)[R], uint32_t xs,
                                           const XOffsets<4>& xo, pk2 (&acc)[R][M]) {
  constexpr int XROW = 64 * Format<FMT_NVFP4>::E;   // bytes between activation rows inside a step
  uint4 wv[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wv[r] = lds128(wrow + woff[r]);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if constexpr (FEW) {
      pk2 xa[M][4], xb[M][4];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        load_x8<XT>(xs + m * XROW + xo.off[2 * h], xa[m]);
        load_x8<XT>(xs + m * XROW + xo.off[2 * h + 1], xb[m]);
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        pk2 wa[4], wb[4];
        decode_e2m1(h ? wv[r].z : wv[r].x, wa);
        decode_e2m1(h ? wv[r].w : wv[r].y, wb);
        const float s = h ? sc[r].y : sc[r].x;
#pragma unroll
        for (int m = 0; m < M; ++m)
          acc[r][m] = ffma2(pack2(s, s), dot16(wa, wb, xa[m], xb[m]), acc[r][m]);
      }
    } else {
      pk2 wa[R][4], wb[R][4];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        decode_e2m1(h ? wv[r].z : wv[r].x, wa[r]);
        decode_e2m1(h ? wv[r].w : wv[r].y, wb[r]);
      }
#pragma unroll
      for (int m = 0; m < M; ++m) {
        pk2 xa[4], xb[4];
        load_x8<XT>(xs + m * XROW + xo.off[2 * h], xa);
        load_x8<XT>(xs + m * XROW + xo.off[2 * h + 1], xb);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float s = h ? sc[r].y : sc[r].x;
          acc[r][m] = ffma2(pack2(s, s), dot16(wa[r], wb[r], xa, xb), acc[r][m]);
        }
      }
    }
  }
}

// The same blocks with the mixed-precision FMA (use_mixed): the rows' weights are brought to the activations' 16-bit
// type once per block (BF16 weights as stored; decoded E4M3 / E2M1 are FP16, exact in BF16 too) and held, the
// activation rows stream past as loaded. Per (row, m): the operations and order of the bodies above.
__device__ __forceinline__ void decode_e4m3_h(uint32_t a, uint32_t b, uint32_t (&h)[4]) {   // 8 E4M3 -> 4 FP16 pairs
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
      : "=r"(h[0]), "=r"(h[1]) : "r"(a));
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
      : "=r"(h[2]), "=r"(h[3]) : "r"(b));
}
__device__ __forceinline__ void decode_e2m1_h(uint32_t a, uint32_t (&h)[4]) {               // 8 E2M1 -> 4 FP16 pairs
  asm("{\n\t.reg .b8 c0, c1, c2, c3;\n\t"
      "mov.b32 {c0, c1, c2, c3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, c0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, c1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, c2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, c3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(a));
}

template <int M, int R>
__device__ __forceinline__ void body_bf16_mixed(uint32_t wrow, const uint32_t (&woff)[R], uint32_t xs, f2 (&acc)[R][M]) {
  constexpr int XROW = 64 * Format<FMT_BF16>::E;
  uint32_t w[R][4];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint4 v = lds128(wrow + woff[r]);
    w[r][0] = v.x; w[r][1] = v.y; w[r][2] = v.z; w[r][3] = v.w;
  }
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const uint4 xv = lds128(xs + m * XROW);
    mixed_rows<__nv_bfloat16, R, M>(w, xv, acc, m);
  }
}

template <int M, int R, typename XT>
__device__ __forceinline__ void body_fp8_mixed(uint32_t wrow, const uint32_t (&woff)[R], uint32_t xs,
                                               const XOffsets<2>& xo, f2 (&acc)[R][M]) {
  constexpr int XROW = 64 * Format<FMT_FP8>::E;
  uint4 wv[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wv[r] = lds128(wrow + woff[r]);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    uint32_t w[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      decode_e4m3_h(j ? wv[r].z : wv[r].x, j ? wv[r].w : wv[r].y, w[r]);
#pragma unroll
      for (int q = 0; q < 4; ++q) w[r][q] = Mixed<XT>::weights(w[r][q]);
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4 xv = lds128(xs + m * XROW + xo.off[j]);
      mixed_rows<XT, R, M>(w, xv, acc, m);
    }
  }
}

// NVFP4: the partial sum of a scale block starts as a product; fma(a, b, -0) is that product bit for bit.
template <int M, int R, typename XT>
__device__ __forceinline__ void body_nvfp4_mixed(uint32_t wrow, const uint32_t (&woff)[R], const float2 (&sc)[R],
                                                 uint32_t xs, const XOffsets<4>& xo, f2 (&acc)[R][M]) {
  constexpr int XROW = 64 * Format<FMT_NVFP4>::E;
  uint4 wv[R];
#pragma unroll
  for (int r = 0; r < R; ++r) wv[r] = lds128(wrow + woff[r]);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t wa[R][4], wb[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      decode_e2m1_h(h ? wv[r].z : wv[r].x, wa[r]);
      decode_e2m1_h(h ? wv[r].w : wv[r].y, wb[r]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        wa[r][q] = Mixed<XT>::weights(wa[r][q]);
        wb[r][q] = Mixed<XT>::weights(wb[r][q]);
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4 xa = lds128(xs + m * XROW + xo.off[2 * h]);
      const uint4 xb = lds128(xs + m * XROW + xo.off[2 * h + 1]);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        f2 part;
        part.lo = -0.0f;
        part.hi = -0.0f;
        part = mixed_fma4<XT>(wa[r], xa, part);
        part = mixed_fma4<XT>(wb[r], xb, part);
        const float s = h ? sc[r].y : sc[r].x;
        acc[r][m].lo = fmaf(s, part.lo, acc[r][m].lo);
        acc[r][m].hi = fmaf(s, part.hi, acc[r][m].hi);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Lane reduction of V values per lane at once: the xor-shuffle tree 16, 8, 4, 2, 1 of every value, with the values
// split between the two partners at each level so that a level costs one shuffle per value pair instead of one per
// value. For each value the additions are those of the plain tree, pair by pair (a + b is commutative in IEEE
// arithmetic), so the bits are the plain tree's. After the last level value v's total sits in lane (v % 32),
// slot v / 32.
template <int V, int OFFSET, int NOUT>
struct LaneReduce {
  static constexpr int H = (V + 1) / 2;   // values kept per lane after this level
  __device__ __forceinline__ static void run(float (&val)[V], int lane, float (&out)[NOUT]) {
    if constexpr (V == 1) {
      float v = val[0];
#pragma unroll
      for (int o = OFFSET; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      out[0] = v;
    } else if constexpr (OFFSET == 0) {
      static_assert(V <= NOUT, "lane reduction output too small");
#pragma unroll
      for (int i = 0; i < V; ++i) out[i] = val[i];
    } else {
      // lanes with the OFFSET bit clear keep values [0, H) and send [H, V); the others keep [H, V) and send [0, H)
      const bool upper = (lane & OFFSET) != 0;
      float keep[H];
#pragma unroll
      for (int i = 0; i < H; ++i) {
        const bool has_hi = H + i < V;
        const float lo = val[i], hi = has_hi ? val[H + i] : 0.0f;
        const float got = __shfl_xor_sync(0xffffffffu, upper ? lo : hi, OFFSET);
        // a value without a partner slot (odd V) is finished by the lower lanes; the upper lanes carry a zero there
        keep[i] = (upper ? hi : lo) + (has_hi || !upper ? got : 0.0f);
      }
      LaneReduce<H, OFFSET / 2, NOUT>::run(keep, lane, out);
    }
  }
};

// Which of the V values lane `lane` holds in output slot `slot` after LaneReduce<V, 16, .> (-1: none).
template <int V>
__device__ __forceinline__ int lane_value(int lane, int slot) {
  int size = V, real = V, base = 0;   // entries [0, real) of this lane's array are values base, base + 1, ...
  for (int o = 16; o > 0; o >>= 1) {
    if (size == 1) return (real == 1 && slot == 0 && (lane & (2 * o - 1)) == 0) ? base : -1;
    const int h = (size + 1) / 2;
    if (lane & o) {
      base += h;
      real = real > h ? real - h : 0;
    } else {
      real = real < h ? real : h;
    }
    size = h;
  }
  return slot < real ? base + slot : -1;
}

// ---------------------------------------------------------------------------------------------------------------
// One tile for one consumer warp holding up to R rows (nr of them real).

// Eight BF16 values as eight FP16 values, and whether each converts exactly (what FP16 holds, its subnormals
// included: the mixed FMA takes subnormal operands exactly, checked on a B200 over every subnormal pattern; values
// beyond 65504 become infinite, NaN compares unequal, and both say no): the test of Arithmetic::HALF_RES.
__device__ __forceinline__ bool bf16x2_fits_half(uint32_t v, uint32_t& h) {
  const float lo = __uint_as_float(v << 16), hi = __uint_as_float(v & 0xffff0000u);
  const __half2 t = __floats2half2_rn(lo, hi);
  h = *reinterpret_cast<const uint32_t*>(&t);
  const float2 back = __half22float2(t);
  return back.x == lo && back.y == hi;
}
__device__ __forceinline__ bool bf16x8_fits_half(const uint4& v, uint4& h) {
  const bool a = bf16x2_fits_half(v.x, h.x), b = bf16x2_fits_half(v.y, h.y);
  const bool c = bf16x2_fits_half(v.z, h.z), d = bf16x2_fits_half(v.w, h.w);
  return a && b && c && d;
}

// Resident activations: the consumer warps bring the whole [M][K] activations into shared memory, once per kernel.
// Warp w takes steps w, w + CW, ...; of a step, lane l holds slots l, l + 32, ... (16 bytes each) of every activation
// row and stores them where a ring stage would have them. BF16 activations (HALF) are tested on the way: the warp
// stores a step as FP16 if all of its values allow it, as loaded otherwise, and says which in the step's flag byte.
// Ends with a barrier of the consumer warps.
template <int FMT, int M, int CW, bool HALF>
__device__ __forceinline__ void fill_resident(const Params& p, unsigned char* smem) {
  constexpr int E = Format<FMT>::E, NQ = E / 8;
  const int nsteps = (p.nblk + 31) >> 5, slots = p.nblk * NQ;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = smem_addr(smem) + (uint32_t)p.x_res_off;
  const uint32_t flags = base + (uint32_t)nsteps * (M * 64 * E);
  const unsigned char* xg = reinterpret_cast<const unsigned char*>(p.x);
  for (int st = warp; st < nsteps; st += CW) {
    uint4 v[M][NQ];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int j = 0; j < NQ; ++j) {
        const int sl = st * (32 * NQ) + j * 32 + lane;
        v[m][j] = sl < slots ? ldg_nc128(xg + (size_t)m * p.ldx * 2 + (size_t)sl * 16) : make_uint4(0u, 0u, 0u, 0u);
      }
    bool fits = false;
    if constexpr (HALF) {
      uint4 h[M][NQ];
      fits = true;
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < NQ; ++j) fits &= bf16x8_fits_half(v[m][j], h[m][j]);   // (slots past the end hold zeros)
      fits = __all_sync(0xffffffffu, fits);
      if (fits) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int j = 0; j < NQ; ++j) v[m][j] = h[m][j];
      }
    }
    const uint32_t dst = base + (uint32_t)st * (M * 64 * E);
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int j = 0; j < NQ; ++j) sts128(dst + m * (64 * E) + swizzle_slot<NQ>(j * 32 + lane) * 16, v[m][j]);
    if (lane == 0) sts_u8(flags + st, fits ? 1u : 0u);
  }
  asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");
}

// The two chains between their two forms (a step that could not be kept as FP16 takes the packed body).
template <int R, int M>
__device__ __forceinline__ void to_packed(const f2 (&a)[R][M], pk2 (&b)[R][M]) {
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) b[r][m] = pack2(a[r][m].lo, a[r][m].hi);
}
template <int R, int M>
__device__ __forceinline__ void from_packed(const pk2 (&b)[R][M], f2 (&a)[R][M]) {
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) asm("mov.b64 {%0, %1}, %2;" : "=f"(a[r][m].lo), "=f"(a[r][m].hi) : "l"(b[r][m].v));
}

template <bool MIXED> struct Chains;   // accumulator pair type of a kernel
template <> struct Chains<false> {
  using type = pk2;
  __device__ __forceinline__ static pk2 zero() { return pack2(0.f, 0.f); }
};
template <> struct Chains<true> {
  using type = f2;
  __device__ __forceinline__ static f2 zero() { f2 z; z.lo = 0.f; z.hi = 0.f; return z; }
};

// SELF: the CTA has no producer warps; its consumer warps share the copies. A warp that has finished iteration `it`
// (stage s) refills the stage of iteration it - 1, which every warp has probably left by then, with iteration
// it + stages - 1: nobody waits for the slowest warp of the iteration just finished, and the ring runs one stage
// short of its depth. All threads share the activation copies; the warps take turns with the weight copies.
template <int FMT, int M, int CW>
__device__ __forceinline__ void self_fill(const Params& p, const Params& maps, const Walk<CW>& wk,
                                          const StageLayout<FMT, M, CW>& lay,
                                          unsigned char* smem, uint32_t full0, uint32_t empty0, int it, int s,
                                          bool with_weights, bool with_activations) {
  const int warp = threadIdx.x >> 5;
  if (with_weights && warp == it % CW)
    Producer<FMT, M, CW, 1>(p, maps, wk, lay, smem, full0, empty0, (int)(threadIdx.x & 31)).weights(it, s);
  if (with_activations)
    Producer<FMT, M, CW, CW>(p, maps, wk, lay, smem, full0, empty0, (int)threadIdx.x).activations_shared(it, s);
}

// RES: the activations are resident (Params::x_resident), not in the stages.
template <int FMT, int M, int R, typename XT, int CW, bool SELF, bool RES = false>
__device__ __forceinline__ bool consume_tile(const Params& p, const Params& maps, const Walk<CW>& wk,
                                             const StageLayout<FMT, M, CW>& lay,
                                             unsigned char* smem, uint32_t full0, uint32_t empty0,
                                             volatile int* abort_flag, int t, int nr, int& s, uint32_t& parity,
                                             int& it) {
  constexpr int E = Format<FMT>::E, SCB = Format<FMT>::SCB, NQ = E / 8;
  constexpr bool FEW = few_rows(FMT, M);
  constexpr bool MIXED = Arithmetic<FMT, M, XT>::MIXED;
  constexpr bool HALF = RES && Arithmetic<FMT, M, XT>::HALF_RES;   // steps flagged as FP16 take the mixed body
  using Acc = typename Chains<MIXED || HALF>::type;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const XOffsets<NQ> xo(lane);
  Acc acc[R][M];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m] = Chains<MIXED || HALF>::zero();
  // Offsets of the warp's rows inside a stage (rows are CW tile rows and one scale group apart); rows the warp does
  // not have alias its last real row (their sums are discarded).
  uint32_t woff[R], scoff[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int rr = min(r, max(nr, 1) - 1);
    woff[r] = (uint32_t)((warp + CW * rr) * lay.w_row + lane * 16);
    scoff[r] = (uint32_t)(lay.sc_off + warp * lay.sc_row + rr * lay.sc_group + (SCB == 64 ? lane * 2 : lane >> 1));
  }
  const bool staged = SCB != 0 && p.scale_mode == SCALES_STAGED;
  const uint32_t ring = smem_addr(smem) + kSmemHeader;
  int rown[R];   // matrix row of each of the warp's rows (rows it does not have alias its last real one)
#pragma unroll
  for (int r = 0; r < R; ++r) {
    int group0, group_n;
    wk.group(t, min(r, max(nr, 1) - 1), group0, group_n);
    rown[r] = group0 + warp;
  }

  // row r's matrix row for an r known only at run time, without indexing the array (it stays in registers)
  auto row_of = [&](int r) {
    int n = rown[0];
#pragma unroll
    for (int q = 1; q < R; ++q) n = r == q ? rown[q] : n;
    return n;
  };

  for (int win = 0; win < wk.nwin; ++win) {
    if (!mbar_wait(full0 + 8u * s, parity, abort_flag)) return false;
    if (it == 0 && threadIdx.x == 0) trace_stamp(p.trace, TRACE_FIRST_FULL);
    if (nr > 0) {
      const uint32_t stage = ring + (uint32_t)s * p.stage_bytes;
      const int blk0 = win * p.steps * 32;
      const int nsteps = min(p.steps, (p.nblk - blk0 + 31) >> 5);
      for (int st = 0; st < nsteps; ++st) {
        const int blk = blk0 + st * 32 + lane;
        if (blk < p.nblk) {
          const uint32_t wrow = stage + st * kStepBytes;
          const int res_step = win * p.steps + st;   // the step's place among the resident ones
          const uint32_t xs = RES ? smem_addr(smem) + (uint32_t)p.x_res_off + (uint32_t)res_step * (M * 64 * E)
                                  : stage + lay.x_off + st * (M * 64 * E);
          bool as_half = false;
          if constexpr (HALF)
            as_half = lds_u8(smem_addr(smem) + (uint32_t)p.x_res_off + (uint32_t)((p.nblk + 31) >> 5) * (M * 64 * E) +
                             res_step) != 0;
          if constexpr (FMT == FMT_BF16) {
            if constexpr (MIXED) body_bf16_mixed<M, R>(wrow, woff, xs + lane * 16, acc);
            else body_bf16<FEW, M, R, XT>(wrow, woff, xs + lane * 16, acc);
          } else if constexpr (FMT == FMT_FP8) {
            if constexpr (MIXED) {
              body_fp8_mixed<M, R, XT>(wrow, woff, xs, xo, acc);
            } else if constexpr (HALF) {
              if (as_half) {
                body_fp8_mixed<M, R, __half>(wrow, woff, xs, xo, acc);
              } else {
                float none[R];
                pk2 packed[R][M];
                to_packed<R, M>(acc, packed);
                body_fp8<FEW, false, M, R, XT>(wrow, woff, none, xs, xo, packed);
                from_packed<R, M>(packed, acc);
              }
            } else {
              float none[R];
              body_fp8<FEW, false, M, R, XT>(wrow, woff, none, xs, xo, acc);
            }
          } else if constexpr (FMT == FMT_MXFP8) {
            float sc[R];
            if (staged) {
#pragma unroll
              for (int r = 0; r < R; ++r) sc[r] = e8m0_to_f32(lds_u8(stage + scoff[r] + st * SCB));
            } else {
#pragma unroll
              for (int r = 0; r < R; ++r) {
                const int n = rown[r];
                sc[r] = e8m0_to_f32(__ldg(p.scales + (size_t)n * p.scale_row_bytes + (blk >> 1)));
              }
            }
            body_fp8<FEW, true, M, R, XT>(wrow, woff, sc, xs, xo, acc);
          } else {
            float2 sc[R];
            if (staged) {
#pragma unroll
              for (int r = 0; r < R; ++r) sc[r] = e4m3x2_to_f32(lds_u16(stage + scoff[r] + st * SCB));
            } else {
#pragma unroll
              for (int r = 0; r < R; ++r) {
                const int n = rown[r];
                const size_t off = p.scale_mode == SCALES_BLOCKED ? tiled_scale_offset(n, blk * 2, p.ct)
                                                                   : (size_t)n * p.scale_row_bytes + blk * 2;
                sc[r] = e4m3x2_to_f32(__ldg(reinterpret_cast<const uint16_t*>(p.scales + off)));
              }
            }
            if constexpr (MIXED) {
              if (HALF && as_half) body_nvfp4_mixed<M, R, __half>(wrow, woff, sc, xs, xo, acc);
              else body_nvfp4_mixed<M, R, XT>(wrow, woff, sc, xs, xo, acc);
            } else if constexpr (HALF) {
              if (as_half) {
                body_nvfp4_mixed<M, R, __half>(wrow, woff, sc, xs, xo, acc);
              } else {
                pk2 packed[R][M];
                to_packed<R, M>(acc, packed);
                body_nvfp4<FEW, M, R, XT>(wrow, woff, sc, xs, xo, packed);
                from_packed<R, M>(packed, acc);
              }
            } else {
              body_nvfp4<FEW, M, R, XT>(wrow, woff, sc, xs, xo, acc);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8u * s);
    if constexpr (SELF) {
      const int next = it + p.stages - 1;
      if (next < wk.ntiles * wk.nwin) {
        const int sp = s == 0 ? p.stages - 1 : s - 1;   // stage of iteration it - 1 (never used yet when it = 0)
        if (it > 0 && !mbar_wait(empty0 + 8u * sp, s == 0 ? parity ^ 1u : parity, abort_flag)) return false;
        self_fill<FMT, M, CW>(p, maps, wk, lay, smem, full0, empty0, next, sp, true, true);
      }
    }
    ++it;
    if (++s == p.stages) { s = 0; parity ^= 1u; }
  }

  // the two chains, then the lanes (xor-shuffle tree 16, 8, 4, 2, 1); scale once; round once
  constexpr int V = R * M;
  float val[V];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) val[r * M + m] = sum2(acc[r][m]);
  float total[(V + 31) / 32];
  LaneReduce<V, 16, (V + 31) / 32>::run(val, lane, total);
  if constexpr (FMT == FMT_NVFP4 && R % 2 == 0) {
    if (p.pairs) {
      // SwiGLU epilogue: the scaled sums of the warp's rows meet in the warp's corner of shared memory behind the
      // ring; lane (j, m) then combines gate row 2 j and up row 2 j + 1 and writes one activation.
      float* meet = reinterpret_cast<float*>(smem + kSmemHeader + (size_t)p.stages * p.stage_bytes) + warp * (RMAX_ALL * 16);
#pragma unroll
      for (int i = 0; i < (V + 31) / 32; ++i) {
        const int v = lane_value<V>(lane, i);
        if (v >= 0) meet[v] = total[i] * __ldg(p.row_scale + row_of(v / M));
      }
      __syncwarp();
      if (lane < (R / 2) * M) {
        const int j = lane / M, m = lane - j * M;
        if (2 * j < nr) {
          const float result = swiglu_value(meet[2 * j * M + m], meet[(2 * j + 1) * M + m]);
          store_out(p.out, p.out_kind, (size_t)m * p.ldo + row_of(2 * j), result);
        }
      }
      __syncwarp();
      return true;
    }
  }
#pragma unroll
  for (int i = 0; i < (V + 31) / 32; ++i) {
    const int v = lane_value<V>(lane, i);
    if (v >= 0) {
      const int r = v / M, m = v - r * M;
      if (r < nr) {
        const int n = row_of(r);
        const float sum = total[i];
        const float result = p.row_scale ? sum * __ldg(p.row_scale + n) : sum;
        if (p.world < 1) {
          store_out(p.out, p.out_kind, (size_t)m * p.ldo + n, result);
        } else {
          store_out(p.out, p.out_kind, ((size_t)p.rank * M + m) * p.ldo + n, result);
        }
      }
    }
  }
  return true;
}

// All-gather epilogue, first half: the CTA's rows [lo, hi) of this rank's slot are complete in the local buffer; all
// consumer threads copy them into the same place of every other rank's buffer: 16 bytes per store where the rows'
// addresses allow it (every rank's buffer has the layout and alignment of this one), else element by element.
template <int M, int CW>
__device__ __forceinline__ void gather_copy(const Params& p) {
  const int tid = threadIdx.x;                       // consumer threads are 0 .. CW * 32 - 1
  asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");
  if (p.world < 2) return;
  const int lo = (int)(((long long)p.N * blockIdx.x) / gridDim.x);
  const int rows = (int)(((long long)p.N * (blockIdx.x + 1)) / gridDim.x) - lo;
  const int esize = p.out_kind == OUT_F32 ? 4 : 2;
  const size_t slot0 = (size_t)p.rank * M * p.ldo + lo;
  bool vector = true;                                // all buffers equally placed within 16 bytes
  for (int q = 0; q < p.world; ++q)
    vector &= ((reinterpret_cast<uintptr_t>(p.peer_out[q]) ^ reinterpret_cast<uintptr_t>(p.out)) & 15) == 0;
  // warp w copies activation rows w, w + CW, ...; its lanes run along the CTA's rows (consecutive addresses)
  const int lane = tid & 31, warp = tid >> 5;
  for (int m = warp; m < M; m += CW) {
    const size_t byte0 = (slot0 + (size_t)m * p.ldo) * esize;
    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.out) + byte0;
    const int bytes = rows * esize;
    // head up to the next 16-byte boundary, 16-byte body, tail
    const int head = vector ? min(bytes, (int)((16 - (reinterpret_cast<uintptr_t>(src) & 15)) & 15)) : bytes;
    const int body = (bytes - head) >> 4;
    for (int i = lane * esize; i < head; i += 32 * esize) {
      if (esize == 4) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(src + i);
        for (int q = 0; q < p.world; ++q)
          if (q != p.rank) *reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(p.peer_out[q]) + byte0 + i) = v;
      } else {
        const uint16_t v = *reinterpret_cast<const uint16_t*>(src + i);
        for (int q = 0; q < p.world; ++q)
          if (q != p.rank) *reinterpret_cast<uint16_t*>(static_cast<unsigned char*>(p.peer_out[q]) + byte0 + i) = v;
      }
    }
    for (int i = lane; i < body; i += 32) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + head + 16 * i);
      for (int q = 0; q < p.world; ++q)
        if (q != p.rank)
          *reinterpret_cast<uint4*>(static_cast<unsigned char*>(p.peer_out[q]) + byte0 + head + 16 * i) = v;
    }
    for (int i = head + 16 * body + lane * esize; i < bytes; i += 32 * esize) {
      if (esize == 4) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(src + i);
        for (int q = 0; q < p.world; ++q)
          if (q != p.rank) *reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(p.peer_out[q]) + byte0 + i) = v;
      } else {
        const uint16_t v = *reinterpret_cast<const uint16_t*>(src + i);
        for (int q = 0; q < p.world; ++q)
          if (q != p.rank) *reinterpret_cast<uint16_t*>(static_cast<unsigned char*>(p.peer_out[q]) + byte0 + i) = v;
      }
    }
  }
}

// Second half: one thread publishes the CTA's copies and counts the CTA done; the rank's last CTA sends `arrivals`
// arrivals to every rank (one per gathered GEMV) and waits, bounded, until its own counter holds arrivals x world.
template <int CW>
__device__ __forceinline__ void gather_signal(const Params& p, volatile int* abort_flag, unsigned int arrivals) {
  asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");
  if (threadIdx.x != 0) return;
  // System-scope operations cost about a microsecond each and this is the kernel's tail, so the chain is kept short:
  // fence (the CTA's peer copies), one acquire-release count per CTA, then the last CTA fences once and sends one
  // relaxed arrival per rank.
  unsigned int* mine = p.peer_flag[p.rank];
  if (p.world > 1) __threadfence_system();           // the CTA's copies, before it counts as done
  unsigned int before;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(before) : "l"(mine + 2) : "memory");
  if (before != gridDim.x - 1) return;
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(mine + 2), "r"(0u) : "memory");   // re-arm the CTA count
  // One system-scope fence orders every CTA's copies (observed through the count) before the arrivals; the
  // arrivals themselves are relaxed, so that they leave back to back (a release per arrival serialised eight
  // round trips on eight GPUs).
  __threadfence_system();
  for (int q = 0; q < p.world; ++q)
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p.peer_flag[q] + p.gather_slot), "r"(arrivals)
                 : "memory");
  if (p.gather_nowait) return;
  const unsigned int want = (unsigned int)p.world * arrivals;
  const unsigned long long start = global_ns();
  bool done = false;
  for (unsigned int i = 1; !done; ++i) {
    unsigned int seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + p.gather_slot) : "memory");
    done = seen >= want;
    if (!done && (i & 63u) == 0u && (*abort_flag || global_ns() - start > p.wait_limit_ns)) break;
  }
  if (done)
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(mine + p.gather_slot), "r"(0u - want) : "memory");
  else if (p.status)
    atomicOr(p.status, kStatusGatherTimeout);
}

// The consumer warps' walk over one GEMV: tiles in order, each for up to RMAX rows a warp. The ring position (s,
// parity) carries over; `fresh`: the ring is empty and unfilled (a kernel's first GEMV, or any GEMV of a kernel
// whose consumers feed themselves, which starts after all its warps have left the previous one).
template <int FMT, int M, typename XT, int CW, bool SELF>
__device__ __forceinline__ bool consume_gemv(const Params& p, const Params& maps, unsigned char* smem, uint32_t full0,
                                             uint32_t empty0, volatile int* abort_flag, int& s, uint32_t& parity,
                                             bool first) {
  constexpr int RMAX = rows_max(FMT, M);
  const int warp = threadIdx.x >> 5;
  const Walk<CW> wk(p);
  const StageLayout<FMT, M, CW> lay(p);
  if constexpr (SELF) {
    // the first stages - 1 iterations, into the stages after s; with static weights, in a kernel's first GEMV, their
    // weight copies leave before the previous kernel of the stream has completed
    const int ahead = min(p.stages - 1, wk.ntiles * wk.nwin);
    const bool early = first && p.early_weights;
    if (early)
      for (int i = 0; i < ahead; ++i)
        self_fill<FMT, M, CW>(p, maps, wk, lay, smem, full0, empty0, i, (s + i) % p.stages, true, false);
    if (first) griddep_wait();
    for (int i = 0; i < ahead; ++i)
      self_fill<FMT, M, CW>(p, maps, wk, lay, smem, full0, empty0, i, (s + i) % p.stages, !early, true);
  } else if (first) {
    griddep_wait();   // consumers read scales and write results in global memory: after the previous kernel
  }
  bool resident = false;
  if constexpr (resident_capable(FMT, M) && !SELF) {
    resident = p.x_resident != 0;
    if (resident) {
      // (a later GEMV of a batch: nobody reads the previous one's activations any more)
      if (!first) asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");
      fill_resident<FMT, M, CW, Arithmetic<FMT, M, XT>::HALF_RES>(p, smem);
    }
  }
  if (first && threadIdx.x == 0) trace_stamp(p.trace, TRACE_DEP);
  int it = 0;
  bool ok = true;
  for (int t = 0; t < wk.ntiles && ok; ++t) {
    int nr = 0;                      // rows this warp holds in the tile: one per group that reaches it
    for (int g = 0; g < p.rows_per_warp; ++g) {
      int group0, group_n;
      wk.group(t, g, group0, group_n);
      if (warp < group_n) nr = g + 1;
    }
    // three rows have their own code only where tiles of odd heights are made on purpose (split tails)
    constexpr bool THREE = M == 1 && RMAX == 4;
    auto tile = [&](auto res) {
      constexpr bool RES = decltype(res)::value;
      if (nr > (THREE ? 3 : 2))
        return consume_tile<FMT, M, RMAX, XT, CW, SELF, RES>(p, maps, wk, lay, smem, full0, empty0, abort_flag, t, nr, s,
                                                             parity, it);
      if (THREE && nr > 2)
        return consume_tile<FMT, M, THREE ? 3 : RMAX, XT, CW, SELF, RES>(p, maps, wk, lay, smem, full0, empty0, abort_flag,
                                                                        t, nr, s, parity, it);
      if (nr > 1)
        return consume_tile<FMT, M, 2, XT, CW, SELF, RES>(p, maps, wk, lay, smem, full0, empty0, abort_flag, t, nr, s,
                                                          parity, it);
      return consume_tile<FMT, M, 1, XT, CW, SELF, RES>(p, maps, wk, lay, smem, full0, empty0, abort_flag, t, nr, s, parity,
                                                        it);
    };
    if constexpr (resident_capable(FMT, M) && !SELF) ok = resident ? tile(std::true_type()) : tile(std::false_type());
    else ok = tile(std::false_type());
  }
  if (!ok && (threadIdx.x & 31) == 0 && p.status) atomicOr(p.status, kStatusConsumerTimeout);
  return ok;
}

// Barriers and the abort word of a CTA; the first thread sets them up.
template <int CW, int COPY_WARPS>
__device__ __forceinline__ void ring_setup(const Params& p, uint32_t full0, uint32_t empty0, volatile int* abort_flag) {
  if (threadIdx.x == 0) {
    if (p.trace) {
      unsigned int sm;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
      p.trace[(size_t)blockIdx.x * kTraceSlots + TRACE_SM] = sm;
      trace_stamp(p.trace, TRACE_ENTRY);
    }
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full0 + 8u * s, 32 * COPY_WARPS + 1);   // the copying lanes' cp.async arrivals + the expect_tx arrival
      mbar_init(empty0 + 8u * s, CW);
    }
    *abort_flag = 0;
    *reinterpret_cast<volatile unsigned long long*>(abort_flag + 2) = p.wait_limit_ns;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  griddep_launch_dependents();
}

template <int FMT, int M, typename XT>
__global__ void __launch_bounds__((consumer_warps(FMT, M) + producer_warps(FMT, M)) * 32, ctas_per_sm(FMT, M))
    gemv_kernel(const __grid_constant__ Params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int CW = consumer_warps(FMT, M), PW = producer_warps(FMT, M);
  constexpr bool SELF = PW == 0;             // no producer warps: the consumers issue the copies themselves
  constexpr int COPY_WARPS = SELF ? CW : PW;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
  const uint32_t full0 = smem_addr(bars), empty0 = full0 + 8u * kMaxStages;
  ring_setup<CW, COPY_WARPS>(p, full0, empty0, abort_flag);
  int s = 0;
  uint32_t parity = 0;
  if ((int)(threadIdx.x >> 5) >= CW) {
    if constexpr (!SELF)
      Producer<FMT, M, CW, COPY_WARPS>(p, p, smem, full0, empty0, (int)threadIdx.x - CW * 32).run(abort_flag, s, parity,
                                                                                                  true);
  } else {
    consume_gemv<FMT, M, XT, CW, SELF>(p, p, smem, full0, empty0, abort_flag, s, parity, true);
    if ((threadIdx.x & 31) == 0) trace_stamp(p.trace, TRACE_LAST_CONSUMED);
    if (p.world >= 1) {
      gather_copy<M, CW>(p);
      gather_signal<CW>(p, abort_flag, 1u);
    }
  }
  if ((threadIdx.x & 31) == 0) trace_stamp(p.trace, TRACE_EXIT);
  // A wait that ran out leaves copies in flight towards this CTA's shared memory: let them land before the CTA's
  // memory is handed to the next one (bounded sleep, error path only).
  if (*abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
}

// Several independent GEMVs of one format and row count in one launch: `items` (device memory) are their launch
// parameters, all with the same ring shape (stages, stage bytes). Every CTA walks the GEMVs in order and the ring never
// drains between them: the copies of the next GEMV's weights are in flight while the last tiles of this one are
// consumed, which a sequence of launches cannot do (a CTA that holds the SM's shared memory must leave before the
// next kernel's CTA can come). With the all-gather epilogue each CTA sends a GEMV's rows to the peers as soon as it has
// finished them and goes on; the arrivals of all GEMVs are exchanged once, at the end. For GEMVs whose inputs do not
// depend on each other's outputs only (all activations are read after one wait for the previous kernel).
template <int FMT, int M, typename XT>
__global__ void __launch_bounds__((consumer_warps(FMT, M) + producer_warps(FMT, M)) * 32, ctas_per_sm(FMT, M))
    gemv_batch_kernel(const Params* __restrict__ items, int count) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int CW = consumer_warps(FMT, M), PW = producer_warps(FMT, M);
  constexpr bool SELF = PW == 0;
  constexpr int COPY_WARPS = SELF ? CW : PW;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
  const uint32_t full0 = smem_addr(bars), empty0 = full0 + 8u * kMaxStages;
  ring_setup<CW, COPY_WARPS>(items[0], full0, empty0, abort_flag);
  int s = 0;
  uint32_t parity = 0;
  if ((int)(threadIdx.x >> 5) >= CW) {
    if constexpr (!SELF) {
      bool ok = true;
      for (int g = 0; g < count && ok; ++g)
        ok = Producer<FMT, M, CW, COPY_WARPS>(items[g], items[g], smem, full0, empty0, (int)threadIdx.x - CW * 32)
                 .run(abort_flag, s, parity, g == 0);
    }
  } else {
    bool ok = true;
    // Where the consumers feed themselves every warp of the CTA is on the same GEMV, and the kernels are short of
    // registers: the GEMV's parameters are then kept in shared memory behind the ring (a read from there costs less
    // than one from global memory; a kernel parameter would cost nothing, but a batch does not fit there).
    Params* held = reinterpret_cast<Params*>(smem + kSmemHeader + (size_t)items[0].stages * items[0].stage_bytes);
    for (int g = 0; g < count && ok; ++g) {
      if constexpr (SELF) {
        asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");
        const uint32_t* src = reinterpret_cast<const uint32_t*>(items + g);
        for (int i = threadIdx.x; i < (int)(sizeof(Params) / 4); i += CW * 32) reinterpret_cast<uint32_t*>(held)[i] = src[i];
        asm volatile("bar.sync 1, %0;" ::"r"(CW * 32) : "memory");
      }
      const Params& p = SELF ? *held : items[g];
      ok = consume_gemv<FMT, M, XT, CW, SELF>(p, items[g], smem, full0, empty0, abort_flag, s, parity, g == 0);
      // the CTA's rows of this GEMV go to the peers now (and, without producer warps, every warp has left the ring
      // before the next GEMV refills it: the copy starts with a barrier of the consumer warps)
      if (p.world >= 1 || SELF) gather_copy<M, CW>(p);
    }
    if ((threadIdx.x & 31) == 0) trace_stamp(items[0].trace, TRACE_LAST_CONSUMED);
    if (items[0].world >= 1) gather_signal<CW>(items[0], abort_flag, (unsigned int)count);
  }
  if ((threadIdx.x & 31) == 0) trace_stamp(items[0].trace, TRACE_EXIT);
  if (*abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
}

}  // namespace dg
