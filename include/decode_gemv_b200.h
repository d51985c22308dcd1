/* C ABI of the B200 decode-GEMV library (libdecode_gemv_b200.so).
 *
 * These entry points are what a binding for the reference package decode-gemv would call in place of its raw CUDA API
 * (decode-gemv/decode_gemv_cuda/decode_gemv.h:30-43): plain pointers and sizes, device pointers unless said otherwise,
 * a cudaStream_t passed as void*. Every function returns a cudaError_t value as int (0 = cudaSuccess;
 * 1 = cudaErrorInvalidValue for a shape, alignment or row-count the kernels cannot read). Nothing allocates, nothing
 * waits for the device: the enqueue calls can be captured in a CUDA graph, as the reference's can (binding.cu:1-2).
 *
 * Common rules (the reference's, binding.cu:19-63 and decode_gemv.cu:382, 396, 405):
 *   x      [M][K] BF16 (x_is_bf16 = 1) or FP16 (0), rows ldx elements apart, ldx % 8 == 0, base on 16 bytes, M 1..16
 *   out    [M][N], rows ldo elements apart; out_kind 0 = FP32, 1 = x's 16-bit type
 *   a row's result is the same bits whatever M is and whatever other rows the matrix holds (summation order is a
 *   function of K and the format only), so an N-slice of a matrix gives the bits of the whole matrix's rows.
 */
#ifndef DECODE_GEMV_B200_H_
#define DECODE_GEMV_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DG_MAX_ROWS 16

#if defined(__GNUC__)
#define DG_API __attribute__((visibility("default")))
#else
#define DG_API
#endif

/* NVFP4 W4A16. Replaces enqueue_gemv (decode_gemv.h:30-32, decode_gemv.cu:378-392).
 * out[m][n] = inverse[n] * sum_k x[m][k] * e2m1(codes[n][k]) * e4m3(scales[n][k / 16])
 * codes [N][K/2] bytes on 16 bytes (element 2i in the low nibble of byte i), K % 32 == 0, K >= 32;
 * scales E4M3 bytes on 2 bytes: row major [N][K/16], or (blocked = 1) cuBLASLt's 128 x 4 tiles with rows padded to
 * 128 and blocks to 4; inverse [N] FP32. */
DG_API int dg_enqueue_nvfp4(const void* x, int ldx, int x_is_bf16, const uint8_t* codes, const uint8_t* scales, int blocked,
                     const float* inverse, void* out, int ldo, int out_kind, int M, int N, int K, void* stream);

/* NVFP4 GEMV of one rank's slice of the output columns with the all-gather fused into the kernel's epilogue. No
 * counterpart in the reference (it has no multi-GPU code); it is the column-sharded stack's replacement for "GEMV,
 * then NCCL all-gather". All `world` ranks (1..8, one GPU each, peers mapped into each other's address space) call
 * it in the same order with the same M, N (rows of this rank's slice), K and slot. peer_out[q] is rank q's gathered
 * buffer [world][M][N] (FP32 or x's type) and peer_flags[q] rank q's block of four zero-initialised 32-bit counters, both
 * as addresses valid on the calling device (host arrays of `world` pointers, read during the call). The kernel stores
 * its [M][N] results into slot `rank` of every rank's buffer, counts the rank in on every rank's counter `slot`, and
 * ends only when every rank's results have arrived in this rank's buffer (bounded wait: dg_take_status bit 2 on
 * time-out). Consecutive calls alternate slot 0 and 1. With slot 2 or 3 the kernel uses counter slot - 2 and does
 * not wait: it only delivers its results and counts the rank in, so that GEMVs whose inputs do not depend on the
 * gathered outputs overlap their gathers; dg_enqueue_gather_wait then collects the arrivals.
 * When a gathered buffer may be written again: a rank starts storing call n + 1's results into its peers' buffers
 * as soon as its own call n has ended, which only says that every rank has FINISHED COMPUTING call n, not that the
 * peers have finished READING what call n gathered. So a buffer that call n filled must not be the target of call
 * n + 1: alternate two buffers (as the counters alternate), after which call n + 2 may reuse the first, because no
 * rank can start it before every rank has passed call n + 1, which is stream-ordered after that rank's readers of
 * call n. With the signal-only form the same holds per collected batch: reuse a buffer only after every rank has
 * passed a later waiting call or dg_enqueue_gather_wait (two sets of buffers, used in turn, satisfy it).
 * After a time-out (status bit 2) the counters hold stray arrivals: re-zero them on every rank (dg_reset_counters)
 * once all ranks are idle, before the next call. */
DG_API int dg_enqueue_nvfp4_allgather(const void* x, int ldx, int x_is_bf16, const uint8_t* codes, const uint8_t* scales,
                                      int blocked, const float* inverse, void* const* peer_out,
                                      void* const* peer_flags, int world, int rank, int slot, int out_kind, int M,
                                      int N, int K, void* stream);

/* Collects the arrivals of all-gather calls made with slot 2 or 3: enqueues a one-thread kernel that waits (bounded,
 * dg_take_status bit 2 on time-out) until counter `slot` (0 or 1) of this rank's block `flags` holds `expected` =
 * (calls made on that counter) x world arrivals and takes them off. When it has run, the results of all those calls
 * from every rank are in this rank's buffers. No counterpart in the reference. */
DG_API int dg_enqueue_gather_wait(void* flags, int slot, unsigned int expected, void* stream);

/* Zeroes a block of four counters in stream order (after a time-out, or before first use of memory that was not
 * zero-filled). Every rank does this for its own block while no all-gather call of the group is in flight. No
 * counterpart in the reference. */
DG_API int dg_reset_counters(void* flags, void* stream);

/* dg_enqueue_nvfp4_allgather for callers that cannot allocate device memory. No counterpart in the reference.
 *
 * Who needs it: a serving process that hands all of HBM to its own weight and KV-cache arenas at start-up and has
 * nothing left for cudaMalloc afterwards; a plugin host or a latency-critical decode loop that forbids allocation
 * after initialisation because cudaMalloc synchronises the device and can fail; code that only learns it needs the
 * counters while a stream is being captured. Such callers own the gathered output buffers already, but have no
 * memory for the arrival counters the fused all-gather needs. Here the counters are DG_NOALLOC_CHANNELS blocks of four built
 * into the library (1 KB on every GPU that loads it, until the process exits); this call and everything under
 * it calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Arguments as dg_enqueue_nvfp4_allgather, except that instead of peer_flags the caller names the CUDA device
 * ordinal of every rank (devices[q], host array of `world` ints) and a channel 0 .. DG_NOALLOC_CHANNELS - 1; rank q's
 * counters are block `channel` in device devices[q]'s copy of the library's array, so all ranks must live in
 * this process (one thread or stream per GPU) with peer access enabled between their devices; world = 1 needs
 * neither. devices[rank] must be the current device. Only the waiting forms exist here (slot 0 or 1): arrivals
 * left by a signal-only call could not be collected, since the built-in counters have no address the caller could
 * hand to dg_enqueue_gather_wait. More than 8 ranks, a channel outside the range, slot 2 or 3, or a current device
 * other than devices[rank] is refused with cudaErrorInvalidValue (1).
 * The first call that names a device looks up that device's array (cudaSetDevice + cudaGetSymbolAddress, then back):
 * make that first call outside any stream capture, and only name devices this process has already initialised
 * (cudaSetDevice on a device without a context creates one, which allocates).
 * Every call on a channel shares its counters, which keep whatever the last call left: a completed call leaves
 * them zero, and that is the state the next call requires. Two calls on the same channel that overlap on the GPU, or a
 * call after one that timed out (dg_take_status bit 2), race on the counters; use another channel, or order them. */
#define DG_NOALLOC_CHANNELS 64
DG_API int dg_enqueue_nvfp4_allgather_noalloc(const void* x, int ldx, int x_is_bf16, const uint8_t* codes,
                                              const uint8_t* scales, int blocked, const float* inverse,
                                              void* const* peer_out, const int* devices, int world, int rank,
                                              int channel, int slot, int out_kind, int M, int N, int K, void* stream);

/* Zeroes the current device's counters of a built-in channel in stream order: the way back to a usable channel after
 * a call on it timed out (dg_take_status bit 2). Every rank calls it for its own device while the group is idle.
 * Allocates nothing. No counterpart in the reference. */
DG_API int dg_reset_noalloc_channel(int channel, void* stream);

/* SwiGLU between the gate_up and down projections: out[row][k] = silu(gate_up[row][k]) * gate_up[row][inter + k]
 * (gate in columns [0, inter), up in [inter, 2 inter), rows ldg elements apart; out rows ldo apart), FP32 arithmetic
 * in the reference's declared operations (x / (1 + exp(-x)) with its polynomial exp), inputs and outputs FP32
 * (in_is_f32 / out_is_f32 = 1) or BF16 (0; one rounding). With FP32 in and out, contiguous, it replaces enqueue_swiglu
 * of the reference's int-block-experts package (int_block_cuda/int_block.h:65, int_block.cu:275-282, :326-331) bit for
 * bit. No allocation, no host synchronisation. */
DG_API int dg_enqueue_swiglu(const void* gate_up, long long ldg, int in_is_f32, int rows, int inter, void* out,
                             long long ldo, int out_is_f32, void* stream);

/* The gate_up projection with SwiGLU in its epilogue: the NVFP4 matrix holds 2 I rows, gate rows [0, I) and up rows
 * [I, 2 I) (codes [2 I][K / 2], scales, inverse [2 I] as dg_enqueue_nvfp4), and out [M][ldo] receives the I activations
 * of the down projection, out[m][k] = silu(g) * u with g, u the two finished FP32 sums times their inverse scales, in the
 * arithmetic of dg_enqueue_swiglu, rounded once to out's type (out_kind 0 FP32, 1 x's type). A warp holds row k of both
 * halves side by side, so nothing but the activations is written: no [M][2 I] intermediate, no second launch. The bits
 * are those of dg_enqueue_nvfp4 with FP32 output followed by dg_enqueue_swiglu. No counterpart in the reference (it
 * runs the steps as separate kernels: int_block.cu:275-282 is its SwiGLU). */
DG_API int dg_enqueue_nvfp4_gate_up_swiglu(const void* x, int ldx, int x_is_bf16, const uint8_t* codes,
                                           const uint8_t* scales, int blocked, const float* inverse, void* out, int ldo,
                                           int out_kind, int M, int I, int K, void* stream);

/* Several NVFP4 GEMVs in one launch. No counterpart in the reference. For projections whose inputs do not depend on each
 * other's outputs (q, k and v; gate and up; a benchmark's independent calls): one persistent kernel walks the GEMVs in
 * order and never lets its stream of weights drain between them, which back-to-back launches cannot do, and with
 * world >= 1 every GEMV's rows go to the peers as soon as a CTA has finished them, the arrivals of all GEMVs being
 * exchanged once at the end of the launch (same buffers, counters, slots and reuse rule as
 * dg_enqueue_nvfp4_allgather; world = 0: no gather, results to out / ldo). Every row has the bits it gets from
 * dg_enqueue_nvfp4. All GEMVs share x's type (BF16 only), M and out_kind.
 *   dg_batch_blob_bytes(count)   bytes of the encoded batch
 *   dg_encode_nvfp4_batch(...)   host only: checks the GEMVs as dg_enqueue_nvfp4 does and writes their launch
 *                                parameters into host_blob, for a copy that will live at device_blob (device memory on
 *                                256 bytes, of the current device). The caller copies host_blob there (once: weights
 *                                and buffers of a decode stack do not move) and keeps host_blob for the enqueue. The
 *                                process-wide settings (static weights, wait limit) are read here.
 *   dg_enqueue_batch(host_blob)  launches the batch on the stream; allocates nothing, waits for nothing. */
typedef struct DgNvfp4BatchItem {
  const void* x;             /* [M][K] BF16, rows ldx apart */
  const uint8_t* codes;      /* as dg_enqueue_nvfp4 */
  const uint8_t* scales;
  const float* inverse;
  void* out;                 /* world = 0: [M][ldo] */
  void* const* peer_out;     /* world >= 1: host array of `world` gathered buffers [world][M][N] */
  int ldx, ldo, blocked, N, K;
} DgNvfp4BatchItem;
DG_API unsigned long long dg_batch_blob_bytes(int count);
DG_API int dg_encode_nvfp4_batch(const DgNvfp4BatchItem* items, int count, int x_is_bf16, int out_kind, int M, int world,
                                 int rank, void* const* peer_flags, int slot, const void* device_blob, void* host_blob);
DG_API int dg_enqueue_batch(const void* host_blob, void* stream);

/* FP8 E4M3 W8A16. Replaces enqueue_gemv_fp8 (decode_gemv.h:34-36, decode_gemv.cu:402-417).
 * Exactly one of row_scale ([N] FP32: out = row_scale[n] * sum) and mx_scale ([N][K/32] E8M0 bytes, MXFP8:
 * each weight times 2^(e - 127)) is non-null. codes [N][K] bytes on 16 bytes, K % 16 == 0 (32 for MXFP8), K >= 16. */
DG_API int dg_enqueue_fp8(const void* x, int ldx, int x_is_bf16, const uint8_t* codes, const float* row_scale,
                   const uint8_t* mx_scale, void* out, int ldo, int out_kind, int M, int N, int K, void* stream);

/* BF16 weights. Replaces enqueue_gemv_bf16 (decode_gemv.h:38-39, decode_gemv.cu:394-400).
 * w [N][K] BF16 on 16 bytes, K % 8 == 0, K >= 8; x BF16; out_kind 0 = FP32, 1 = BF16. */
DG_API int dg_enqueue_bf16(const void* x, int ldx, const void* w, void* out, int ldo, int out_kind, int M, int N, int K,
                    void* stream);

/* NVFP4 dequantizer: the matrix's values [N][K], contiguous, as BF16 (out_kind 1), FP16 (2) or FP8 E4M3 (3):
 * e2m1(code) * scale (exact in FP32) times factor[row], one FP32 product, rounded once to the output type; the FP8
 * form saturates at +-448 (the row's values in units of the caller's per-row scale, factor = inverse / that scale).
 * Replaces the reference package's Triton dequantizers decode and decode_fp8 (torch-ext/decode_gemv/
 * triton_gemv.py:171-176 and :195-200, kernels :156-168 and :179-192; contract pinned by
 * tests/test_decode_gemv.py:131-140). codes [N][K/2] and out on 16 bytes, scales [N][K/16] E4M3 row-major,
 * factor [N] FP32, K % 16 == 0, K >= 16, N >= 1. No allocation, no host synchronisation. */
DG_API int dg_enqueue_dequantize(const uint8_t* codes, const uint8_t* scales, const float* factor, void* out,
                                 int out_kind, int N, int K, void* stream);

/* Activation quantizer, FP8 per row: q [M][K] E4M3 bytes (rows ldq bytes apart) and scale [M] FP32 from x [M][K] BF16
 * (rows ldx elements apart): scale = max(amax * fp32(1 / 448), 1e-12), q = E4M3(clamp(x / scale, +-448)), IEEE
 * division, round to nearest even; a NaN in a row makes its scale NaN. Any M >= 1 and K >= 1; rows on 16 bytes with
 * K % 8 == 0 are read from HBM once (staged in shared memory), others twice through L2. Replaces
 * enqueue_quantize_fp8_rows of the reference's mma-rows package (mma_rows_cuda/mma_rows.h:109, mma_rows.cu:320-327,
 * kernel :15-90), bit for bit. No allocation, no host synchronisation. */
DG_API int dg_enqueue_quantize_fp8_rows(const void* x, long long ldx, int M, int K, uint8_t* q, long long ldq,
                                        float* scale, void* stream);

/* Activation quantizer, NVFP4: codes [M][K / 2] (element 2i in the low nibble of byte i, on 8 bytes) and E4M3 block
 * scales in cuBLASLt's 128 x 4 tiled layout of [M][K / 16] (rows padded to 128, blocks to 4, the padding written as
 * zero; on 4 bytes) from x [M][K] BF16 (rows on 16 bytes, ldx % 8 == 0), K % 16 == 0, under input scale g =
 * input_scale with input_rcp = 1 / g: per 16 values s = E4M3(min((amax * fp32(1 / 6)) * g, 448)),
 * d = max(e4m3(s) * input_rcp, 1e-30), code = E2M1(x / d) nearest with ties to the even code, saturating at 6, all
 * codes 0 where e4m3(s) is not > 0. Replaces enqueue_quantize_nvfp4 (mma_rows.h:111, mma_rows.cu:329-338, kernel
 * :117-140, arithmetic tile_parts.cuh:57-64 and :309-331), bit for bit. No allocation, no host synchronisation. */
DG_API int dg_enqueue_quantize_nvfp4(const void* x, long long ldx, int M, int K, float input_scale, float input_rcp,
                                     uint8_t* codes, uint8_t* blocked_scales, void* stream);

/* 1 when the current device runs this build's hardware E2M1 conversion (cvt.rn.f16x2.e2m1x2; always, on the sm_100a
 * target this library is built for), -1 when the current device cannot run the library. Replaces hardware_decode
 * (decode_gemv.h:43, decode_gemv.cu:419-427); unlike it, allocates nothing and launches nothing. */
DG_API int dg_hardware_decode(void);

/* The launch a call with these sizes makes, for benches and tests: fmt 0 BF16, 1 FP8, 2 MXFP8, 3 NVFP4.
 * plan[0] = CTAs, [1] = rows per consumer warp and tile, [2] = 512-byte steps per ring stage, [3] = ring stages,
 * [4] = bytes per stage, [5] = dynamic shared memory bytes (256 bytes of barriers, the ring, and, for FP8 / NVFP4 at
 * few rows and small K, the activations, which then stay resident behind the ring for the whole kernel instead of
 * passing through the stages). Host only; returns 0, or 1 for sizes the kernels refuse. */
DG_API int dg_plan(int fmt, int M, int N, int K, int plan[6]);

/* Reads and clears the current device's error word: bit 0 a producer wait ran out, bit 1 a consumer wait ran out,
 * bit 2 a wait for all-gather arrivals ran out (a bounded wait inside a kernel gave up; the call's output is then
 * incomplete). Synchronises the device. Host diagnostic, not part of the hot path; returns the word (0 = clean) or a
 * negative cudaError_t. */
DG_API int dg_take_status(void);

/* Sets how long any wait inside the kernels may last before it gives up (nanoseconds; 0 restores the default of
 * 2 s) and returns the previous limit. Applies to launches enqueued afterwards; process-wide. A serving process
 * that detects a lost peer on the host can keep this short so that the GPU side returns promptly with status bit 2
 * instead of holding the stream for seconds. No counterpart in the reference. */
DG_API unsigned long long dg_set_wait_limit_ns(unsigned long long limit_ns);

/* Tells the library whether weights (codes, block scales staged with them, BF16 weights) are static: not written by
 * any kernel of the stream that can still be in flight when a GEMV starts. Every GEMV kernel is launched with
 * programmatic dependent launch and lets its own successor start at once, so a GEMV may begin while the kernel before
 * it, and in a run of GEMVs the ones before that, are still finishing; it always waits for all of them before it
 * reads activations, row / inverse scales or directly-read block scales and before it writes. With enabled = 1 it
 * starts streaming weights before that wait, which hides its start-up behind the previous kernels' tails (what a
 * decode stack with resident weights wants); with 0 (the default) nothing is read before the wait, which is correct
 * for any caller. The setting is read when a call is enqueued (a captured graph keeps what it was captured with).
 * Process-wide; returns the previous setting, so a caller can scope it. No counterpart in the reference. */
DG_API int dg_set_static_weights(int enabled);

/* Diagnostic: where a launch's time goes. `buffer` is zero-filled device memory for `launches` regions of
 * DG_TRACE_CTAS x DG_TRACE_SLOTS 64-bit words; the i-th GEMV launch after this call (any stream, any format) leaves
 * per CTA c, at word (i * DG_TRACE_CTAS + c) * DG_TRACE_SLOTS + s, the %globaltimer value (ns) at which: s = 0 the
 * CTA started, 1 its wait for the previous kernel of the stream ended, 2 its first ring stage was full, 3 its last
 * consumer warp finished its rows, 4 its last warp left; s = 5 is the SM id. Launches beyond `launches` are not
 * traced; buffer = NULL switches tracing off (the default: the kernels then only test one pointer). Process-wide,
 * host only. No counterpart in the reference. */
#define DG_TRACE_CTAS 320
#define DG_TRACE_SLOTS 8
DG_API int dg_set_trace(void* buffer, int launches);

/* Library version: 100 * major + minor. */
DG_API int dg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DECODE_GEMV_B200_H_ */
