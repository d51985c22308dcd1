// C ABI of the B200 decode GEMVs (include/decode_gemv_b200.h): argument validation, launch planning, dispatch.
//
// Mirrors the reference's raw CUDA API (decode-gemv/decode_gemv_cuda/decode_gemv.cu:378-427): the same refusals
// (cudaErrorInvalidValue for M outside 1..16, N < 1, K not a multiple the format needs, both or neither FP8 scale),
// cudaGetLastError() after the launch, no allocation and no host synchronisation on the enqueue path.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "../../include/decode_gemv_b200.h"
#include "dg_kernel.cuh"
#include "dg_tables.h"

namespace {

using dg::Params;

// Error word the kernels' bounded waits report into: one per device that loads the library.
__device__ int dg_status_word;

constexpr int kMaxDevices = 64;

struct DeviceState {
  std::atomic<int> ready{0};   // 0 unknown, 1 initialised, -1 unusable
  int sms = 0;
  int* status = nullptr;
};

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link against libcuda.
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_tiled() {
  static EncodeTiled fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &found) != cudaSuccess ||
        found != cudaDriverEntryPointSuccess)
      ptr = nullptr;
    return reinterpret_cast<EncodeTiled>(ptr);
  }();
  return fn;
}

// A map over `rows` rows of `row_bytes` bytes (a multiple of 16) as 8-byte elements, box = box_rows x box_bytes.
// The encoded map is a function of these six values alone, and a decode loop asks for the same few maps token after
// token: each host thread keeps the last ones it encoded (the driver call costs about as much as the launch).
bool encode_rows(CUtensorMap* map, const void* base, int rows, int row_bytes, int box_rows, int box_bytes) {
  EncodeTiled fn = encode_tiled();
  if (!fn || row_bytes % 16 || box_bytes % 16 || box_bytes / 8 > 256 || box_rows > 256 || box_rows < 1) return false;
  struct Kept {
    const void* base = nullptr;
    int rows = 0, row_bytes = 0, box_rows = 0, box_bytes = 0;
    CUtensorMap map;
  };
  constexpr int kKept = 64;
  static thread_local Kept kept[kKept];
  const uintptr_t mixed = reinterpret_cast<uintptr_t>(base) >> 8;
  Kept& slot = kept[(mixed ^ (mixed >> 7) ^ (uintptr_t)rows ^ ((uintptr_t)box_rows << 3) ^ (uintptr_t)box_bytes) % kKept];
  if (slot.base == base && slot.rows == rows && slot.row_bytes == row_bytes && slot.box_rows == box_rows &&
      slot.box_bytes == box_bytes) {
    *map = slot.map;
    return true;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  const cuuint32_t box[2] = {(cuuint32_t)(box_bytes / 8), (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  if (fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(base), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  slot.base = base; slot.rows = rows; slot.row_bytes = row_bytes; slot.box_rows = box_rows; slot.box_bytes = box_bytes;
  slot.map = *map;
  return true;
}
DeviceState g_devices[kMaxDevices];
std::atomic<int> g_static_weights{0};   // dg_set_static_weights
std::atomic<unsigned long long> g_wait_limit_ns{dg::kWaitLimitNs};   // dg_set_wait_limit_ns
// dg_set_trace: launch i of the GEMV kernels (counted from the call that set the buffer) stamps into region i
std::atomic<unsigned long long*> g_trace_base{nullptr};
std::atomic<int> g_trace_capacity{0}, g_trace_next{0};

const void* const* const kTables[] = {dg_table_bf16,       dg_table_fp8_bf16,   dg_table_fp8_f16,  dg_table_mxfp8_bf16,
                                      dg_table_mxfp8_f16,  dg_table_nvfp4_bf16, dg_table_nvfp4_f16};

// Per device, once: SM count, the address of the status word, and the opt-in to 227 KB of dynamic shared memory for
// every kernel. None of this is a stream operation. Returns nullptr when the device cannot run sm_100a code.
DeviceState* device_state() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  DeviceState& st = g_devices[dev];
  int ready = st.ready.load(std::memory_order_acquire);
  if (ready == 1) return &st;
  if (ready == -1) return nullptr;
  int major = 0, sms = 0;
  void* status = nullptr;
  bool ok = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess && major == 10 &&
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0 &&
            cudaGetSymbolAddress(&status, dg_status_word) == cudaSuccess;
  // (the carveout preference keeps the SM's whole shared memory available where two CTAs are to share it)
  for (const void* const* table : kTables)
    for (int m = 0; ok && m < 16; ++m)
      ok = cudaFuncSetAttribute(table[m], cudaFuncAttributeMaxDynamicSharedMemorySize, dg::kSmemLimit) == cudaSuccess &&
           cudaFuncSetAttribute(table[m], cudaFuncAttributePreferredSharedMemoryCarveout,
                                cudaSharedmemCarveoutMaxShared) == cudaSuccess;
  for (int m = 0; ok && m < 16; ++m)
    ok = cudaFuncSetAttribute(dg_batch_table_nvfp4_bf16[m], cudaFuncAttributeMaxDynamicSharedMemorySize,
                              dg::kSmemLimit) == cudaSuccess;
  if (!ok) {
    cudaGetLastError();
    st.ready.store(-1, std::memory_order_release);
    return nullptr;
  }
  st.sms = sms;
  st.status = static_cast<int*>(status);
  st.ready.store(1, std::memory_order_release);
  return &st;
}

struct FormatInfo {
  int e, scb;   // elements per 16-byte block, scale bytes per 512-byte step
};
constexpr FormatInfo kFormats[4] = {{8, 0}, {16, 0}, {16, 16}, {32, 64}};

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Launch shape: a speed choice from (format, M, N, K, SM count) only; no row's bits depend on it.
//   CTAs            one per SM, fewer when the matrix has under four rows per SM
//   rows per warp   the most the kernel holds (rows_max), less when a CTA's range is short
//   steps           512-byte steps per ring stage: at least two (1 KB of every row per stage: 512-byte pieces cost
//                   DRAM efficiency and per-row bulk copies are issue-limited), up to four when a tile has few rows;
//                   activations under 32 KB per stage
//   stages          as many as fit in shared memory, at most kMaxStages
// Dynamic shared memory a CTA may take: all of an SM's, or its share where several CTAs live on one SM together
// (the system keeps 1 KB per CTA).
int smem_limit(int fmt, int M) {
  const int share = dg::ctas_per_sm(fmt, M);
  return share == 1 ? dg::kSmemLimit : ((dg::kSmemLimit + 1024) / share - 1024) & ~127;
}

// Bytes of a row's activations kept resident: whole steps of [M][64 * e elements], then a flag byte per step.
int resident_bytes_of(int fmt, int M, int nblk) {
  const int row_steps = ceil_div(nblk, 32);
  return row_steps * M * 64 * kFormats[fmt].e + ((row_steps + 15) & ~15);
}

// `grid` > 0: the launch is a batch's (that many CTAs whatever N; the caller sizes the ring for all its GEMVs and
// decides about resident activations: `allow_resident` is its wish, and no stage rule is applied here).
bool make_plan(int fmt, int M, int N, int K, int sms, Params& p, int& ctas, int& smem, int grid = 0,
               bool allow_resident = true) {
  const FormatInfo f = kFormats[fmt];
  const int cw = dg::consumer_warps(fmt, M);
  const long long row_bits = (long long)K * 128 / f.e;   // 16 bytes per e elements
  p.row_bytes = (int)(row_bits / 8);
  p.nblk = p.row_bytes / 16;
  const int share = dg::ctas_per_sm(fmt, M);   // CTAs that live on one SM together
  sms *= share;
  ctas = grid > 0 ? grid : sms < ceil_div(N, 4) ? sms : ceil_div(N, 4);   // grid: the launch is shared (batch)
  const int rows_per_cta = ceil_div(N, ctas);
  const int per_warp = ceil_div(rows_per_cta, cw);
  int rmax = dg::rows_max(fmt, M);
  // Tuning aid: DG_FORCE_PLAN="rows,steps" caps the rows per warp and fixes the steps per stage (read once).
  static const char* forced = std::getenv("DG_FORCE_PLAN");
  int force_rows = 0, force_steps = 0;
  if (forced && std::sscanf(forced, "%d,%d", &force_rows, &force_steps) >= 1 && force_rows >= 1 && force_rows < rmax)
    rmax = force_rows;
  p.rows_per_warp = per_warp < rmax ? per_warp : rmax;
  if (p.pairs) p.rows_per_warp = p.rows_per_warp >= 4 ? 4 : 2;   // gate and up rows side by side: an even count
  const int rows_cap = cw * p.rows_per_warp;
  const int w_step = rows_cap * (dg::kStepBytes + f.scb);   // sizing estimate; the exact stage size is below
  const int row_steps = ceil_div(p.nblk, 32);
  // The ring for activations that pass through the stages (x_step bytes of every step) or stay resident behind it
  // (x_step = 0, resident_bytes taken from the ring's room).
  const int pairs_bytes = p.pairs ? dg::kMeetBytes : 0;   // the SwiGLU epilogue's meeting place, behind the ring
  auto ring = [&](int x_step, int resident_bytes, int& steps, int& stage_bytes) {
    steps = ceil_div(32768, w_step);
    if (steps < 2) steps = 2;
    if (steps > 4) steps = 4;   // a tensor-copy box is at most 256 eight-byte elements (2 KB) wide
    // BF16 rows are the longest per K: 1.5 KB pieces in two deep stages measured up to 14 % faster than 1 KB pieces
    // in three (8192 x 28672, M = 2: 82.9 -> 72.7 us; M = 1 unchanged), FP8 the other way round
    if (fmt == dg::FMT_BF16 && dg::shape_class(fmt, M) == 0 && steps < 3) steps = 3;
    if (steps > row_steps) steps = row_steps;
    while (steps > 1 && steps * x_step > 32768) --steps;
    if (force_steps >= 1) steps = force_steps < row_steps ? force_steps : row_steps;
    if (steps > 8) steps = 8;
    if (steps < 1) steps = 1;
    stage_bytes = (steps * (rows_cap * dg::kStepBytes + x_step) +
                   p.rows_per_warp * dg::scale_group_bytes(cw, steps, f.scb) + 127) & ~127;
    int stages = (smem_limit(fmt, M) - dg::kSmemHeader - pairs_bytes - resident_bytes) / stage_bytes;
    return stages > dg::kMaxStages ? dg::kMaxStages : stages;
  };
  int steps = 0, stage_bytes = 0;
  int stages = ring(M * 64 * f.e, 0, steps, stage_bytes);
  // Activations that are small enough stay in shared memory for the whole kernel instead of passing through the
  // stages, unless that costs the ring its third stage.
  const int resident_bytes = resident_bytes_of(fmt, M, p.nblk);
  p.x_resident = 0;
  // (a batch shares one ring and one resident area between GEMVs of different K: only the smaller ones stay resident)
  if (allow_resident && dg::resident_capable(fmt, M) &&
      resident_bytes <= (grid > 0 ? dg::kResidentLimit / 2 - 15 * 1024 : dg::kResidentLimit)) {
    int steps_r = 0, stage_bytes_r = 0;
    const int stages_r = ring(0, resident_bytes, steps_r, stage_bytes_r);
    if (grid > 0 || stages_r >= 3 || stages_r >= stages) {
      p.x_resident = 1;
      steps = steps_r; stage_bytes = stage_bytes_r; stages = stages_r;
    }
  }
  if (stages < 2) return false;
  p.steps = steps;
  p.stage_bytes = stage_bytes;
  p.stages = stages;
  p.x_res_off = dg::kSmemHeader + stages * stage_bytes + pairs_bytes;
  smem = p.x_res_off + (p.x_resident ? resident_bytes : 0);
  return true;
}

bool aligned(const void* ptr, uintptr_t bytes) { return reinterpret_cast<uintptr_t>(ptr) % bytes == 0; }

// Everything of a launch but the launch: plan, tensor maps, process-wide settings. `grid` > 0 fixes the CTA count.
int prepare(int fmt, Params& p, int M, int& ctas, int& smem, int grid = 0, bool allow_resident = true) {
  DeviceState* st = device_state();
  if (!st) return (int)cudaErrorInvalidDevice;
  if (!make_plan(fmt, M, p.N, p.K, st->sms, p, ctas, smem, grid, allow_resident)) return (int)cudaErrorInvalidValue;
  p.status = st->status;
  // Tensor maps for the 2-D copies of full row groups; without them every row travels as a 1-D bulk copy.
  const int cw = dg::consumer_warps(fmt, M);
  const int win_bytes = p.steps * dg::kStepBytes;
  const int matrix_rows = p.pairs ? 2 * p.pairs : p.N;
  p.use_2d = matrix_rows >= cw && encode_rows(&p.tmap_w, p.w, matrix_rows, p.row_bytes, cw, win_bytes);
  if (p.use_2d && p.scale_mode == dg::SCALES_STAGED)
    p.use_2d = encode_rows(&p.tmap_sc, p.scales, matrix_rows, p.scale_row_bytes, cw, p.steps * kFormats[fmt].scb);
  p.early_weights = g_static_weights.load(std::memory_order_relaxed);
  p.wait_limit_ns = g_wait_limit_ns.load(std::memory_order_relaxed);
  static const bool no_split = std::getenv("DG_NO_SPLIT_TAIL") != nullptr;   // tuning aid
  p.split_tail = M == 1 && !no_split;
  return 0;
}

// Programmatic dependent launch: the kernel may start while the previous kernel of the stream drains (its launch,
// barrier set-up and, with static weights, its first weight copies overlap that tail); it waits for the previous
// kernel before it reads activations or scales from global memory and before it writes.
int launch_pdl(const void* kernel, void** args, int ctas, int threads, int smem, cudaStream_t stream) {
  static const bool no_pdl = std::getenv("DG_NO_PDL") != nullptr;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas);
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = (size_t)smem;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = no_pdl ? 0 : 1;
  const cudaError_t e = cudaLaunchKernelExC(&config, kernel, args);
  return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

int launch(int table, int fmt, Params& p, int M, cudaStream_t stream) {
  int ctas = 0, smem = 0;
  if (const int code = prepare(fmt, p, M, ctas, smem)) return code;
  if (unsigned long long* base = g_trace_base.load(std::memory_order_acquire)) {
    const int index = g_trace_next.fetch_add(1, std::memory_order_relaxed);
    if (index < g_trace_capacity.load(std::memory_order_relaxed))
      p.trace = base + (size_t)index * DG_TRACE_CTAS * dg::kTraceSlots;
  }
  void* args[] = {&p};
  const int threads = 32 * (dg::consumer_warps(fmt, M) + dg::producer_warps(fmt, M));
  return launch_pdl(kTables[table][M - 1], args, ctas, threads, smem, stream);
}

// Argument rules of the NVFP4 GEMV (dg_enqueue_nvfp4) and the fields they determine.
bool fill_nvfp4(Params& p, const void* x, int ldx, int x_is_bf16, const uint8_t* codes, const uint8_t* scales, int blocked,
                const float* inverse, int out_kind, int M, int N, int K) {
  if (M < 1 || M > DG_MAX_ROWS || N < 1 || K < 32 || K % 32) return false;
  if (!x || !codes || !scales || !inverse || ldx % 8 || !aligned(x, 16) || !aligned(codes, 16) || !aligned(scales, 2) ||
      !aligned(inverse, 4) || (out_kind != 0 && out_kind != 1))
    return false;
  p.x = x; p.ldx = ldx; p.w = codes; p.scales = scales; p.row_scale = inverse;
  p.out_kind = out_kind == 0 ? dg::OUT_F32 : (x_is_bf16 ? dg::OUT_BF16 : dg::OUT_F16);
  p.N = N; p.K = K;
  p.scale_row_bytes = K / 16;
  p.ct = blocked ? (K / 16 + 3) / 4 : 0;
  // Scale rows travel by bulk copy when every window of every row starts on 16 bytes and is a multiple of 16 bytes
  // long (K a multiple of 256, base on 16 bytes); otherwise, and for the tiled layout, lanes read them directly.
  p.scale_mode = blocked ? dg::SCALES_BLOCKED
                         : (K % 256 == 0 && aligned(scales, 16)) ? dg::SCALES_STAGED : dg::SCALES_DIRECT;
  return true;
}

// Head of an encoded batch (dg_encode_nvfp4_batch); the GEMVs' launch parameters follow at kBatchHead bytes.
constexpr unsigned int kBatchMagic = 0x44474231u;   // "DGB1"
constexpr size_t kBatchHead = 256;
struct BatchHead {
  unsigned int magic;
  int count, M, ctas, smem, threads, device;
  const void* device_blob;
};
static_assert(sizeof(BatchHead) <= kBatchHead && kBatchHead % alignof(Params) == 0, "batch head layout");

}  // namespace

extern "C" {

int dg_enqueue_nvfp4(const void* x, int ldx, int x_is_bf16, const uint8_t* codes, const uint8_t* scales, int blocked,
                     const float* inverse, void* out, int ldo, int out_kind, int M, int N, int K, void* stream) {
  Params p{};
  if (!out || !fill_nvfp4(p, x, ldx, x_is_bf16, codes, scales, blocked, inverse, out_kind, M, N, K))
    return (int)cudaErrorInvalidValue;
  p.out = out; p.ldo = ldo;
  return launch(x_is_bf16 ? 5 : 6, dg::FMT_NVFP4, p, M, static_cast<cudaStream_t>(stream));
}

int dg_enqueue_nvfp4_allgather(const void* x, int ldx, int x_is_bf16, const uint8_t* codes, const uint8_t* scales,
                               int blocked, const float* inverse, void* const* peer_out, void* const* peer_flags,
                               int world, int rank, int slot, int out_kind, int M, int N, int K, void* stream) {
  Params p{};
  if (!peer_out || !peer_flags || world < 1 || world > dg::kMaxRanks || rank < 0 || rank >= world || slot < 0 ||
      slot > 3 || !fill_nvfp4(p, x, ldx, x_is_bf16, codes, scales, blocked, inverse, out_kind, M, N, K))
    return (int)cudaErrorInvalidValue;
  p.ldo = N;
  p.world = world; p.rank = rank; p.gather_slot = slot & 1; p.gather_nowait = slot >> 1;
  for (int q = 0; q < world; ++q) {
    if (!peer_out[q] || !peer_flags[q] || !aligned(peer_flags[q], 4)) return (int)cudaErrorInvalidValue;
    p.peer_out[q] = peer_out[q];
    p.peer_flag[q] = static_cast<unsigned int*>(peer_flags[q]);
  }
  p.out = peer_out[rank];
  return launch(x_is_bf16 ? 5 : 6, dg::FMT_NVFP4, p, M, static_cast<cudaStream_t>(stream));
}

// Waits (bounded) until counter `slot` of this rank's block holds `expected` arrivals, then takes them off.
__global__ void gather_wait_kernel(unsigned int* counter, unsigned int expected, int* status,
                                   unsigned long long limit_ns) {
  const unsigned long long start = dg::global_ns();
  bool done = false;
  for (unsigned int i = 1; !done; ++i) {
    unsigned int seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(counter) : "memory");
    done = seen >= expected;
    if (!done && (i & 63u) == 0u && dg::global_ns() - start > limit_ns) break;
  }
  if (done) atomicSub_system(counter, expected);
  else if (status) atomicOr(status, dg::kStatusGatherTimeout);
  __threadfence_system();
}

int dg_enqueue_gather_wait(void* flags, int slot, unsigned int expected, void* stream) {
  DeviceState* st = device_state();
  if (!st) return (int)cudaErrorInvalidDevice;
  if (!flags || !aligned(flags, 4) || (slot != 0 && slot != 1) || expected == 0) return (int)cudaErrorInvalidValue;
  gather_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned int*>(flags) + slot, expected,
                                                                    st->status,
                                                                    g_wait_limit_ns.load(std::memory_order_relaxed));
  return (int)cudaGetLastError();
}

int dg_reset_counters(void* flags, void* stream) {
  if (!flags || !aligned(flags, 4)) return (int)cudaErrorInvalidValue;
  return (int)cudaMemsetAsync(flags, 0, 4 * sizeof(unsigned int), static_cast<cudaStream_t>(stream));
}

// ---- the entry point that allocates nothing ---------------------------------------------------------------------
// Arrival counters for dg_enqueue_nvfp4_allgather_noalloc: DG_NOALLOC_CHANNELS blocks of four 32-bit counters that live
// in the library's image on every GPU that loads it (1 KB per GPU, held until the process exits), zero when the
// module is loaded and re-armed to zero by every call that completes. In host code `dg_gather_scratch` is only a
// handle for the runtime, not a device address: the address a kernel may use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
static __device__ __align__(256) unsigned int dg_gather_scratch[4 * DG_NOALLOC_CHANNELS];
static std::atomic<unsigned int*> g_gather_scratch[kMaxDevices];   // per device, filled by the first call that names it

static cudaError_t gather_scratch_of(int device, unsigned int** out) {
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  if (!g_gather_scratch[device].load(std::memory_order_acquire)) {
    int previous = 0;
    cudaError_t e = cudaGetDevice(&previous);
    if (e == cudaSuccess && previous != device) e = cudaSetDevice(device);
    void* address = nullptr;
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&address, dg_gather_scratch);
    if (previous != device) {
      const cudaError_t back = cudaSetDevice(previous);
      if (e == cudaSuccess) e = back;
    }
    if (e != cudaSuccess) return e;
    g_gather_scratch[device].store(static_cast<unsigned int*>(address), std::memory_order_release);
  }
  *out = g_gather_scratch[device].load(std::memory_order_acquire);
  return cudaSuccess;
}

int dg_enqueue_nvfp4_allgather_noalloc(const void* x, int ldx, int x_is_bf16, const uint8_t* codes,
                                       const uint8_t* scales, int blocked, const float* inverse,
                                       void* const* peer_out, const int* devices, int world, int rank, int channel,
                                       int slot, int out_kind, int M, int N, int K, void* stream) {
  if (!devices || world < 1 || world > dg::kMaxRanks || channel < 0 || channel >= DG_NOALLOC_CHANNELS)
    return (int)cudaErrorInvalidValue;   // more ranks or channels than the built-in counters cover
  // Only the waiting forms: a signal-only call (slot 2, 3) would leave arrivals on counters that no caller can
  // reach to collect, and the channel's next waiting call would then end before its data has landed.
  if (slot != 0 && slot != 1) return (int)cudaErrorInvalidValue;
  int current = -1;
  if (rank < 0 || rank >= world || cudaGetDevice(&current) != cudaSuccess || current != devices[rank])
    return (int)cudaErrorInvalidValue;   // the kernel counts its CTAs on the current device's block
  void* flags[dg::kMaxRanks];
  for (int q = 0; q < world; ++q) {
    unsigned int* base = nullptr;
    const cudaError_t e = gather_scratch_of(devices[q], &base);
    if (e != cudaSuccess) return (int)e;
    flags[q] = base + 4 * channel;
  }
  return dg_enqueue_nvfp4_allgather(x, ldx, x_is_bf16, codes, scales, blocked, inverse, peer_out, flags, world, rank,
                                    slot, out_kind, M, N, K, stream);
}

int dg_enqueue_nvfp4_gate_up_swiglu(const void* x, int ldx, int x_is_bf16, const uint8_t* codes, const uint8_t* scales,
                                    int blocked, const float* inverse, void* out, int ldo, int out_kind, int M, int I,
                                    int K, void* stream) {
  Params p{};
  if (!out || I < 1 || I > (1 << 29) ||
      !fill_nvfp4(p, x, ldx, x_is_bf16, codes, scales, blocked, inverse, out_kind, M, 2 * I, K))
    return (int)cudaErrorInvalidValue;
  p.out = out; p.ldo = ldo;
  p.pairs = I;
  // the tiles walk whole blocks of gate rows and up rows in turn: N counts the rows in that order
  const int cw = dg::consumer_warps(dg::FMT_NVFP4, M);
  p.N = 2 * ((I + cw - 1) / cw) * cw;
  return launch(x_is_bf16 ? 5 : 6, dg::FMT_NVFP4, p, M, static_cast<cudaStream_t>(stream));
}

unsigned long long dg_batch_blob_bytes(int count) { return count > 0 ? kBatchHead + (size_t)count * sizeof(Params) : 0; }

int dg_encode_nvfp4_batch(const DgNvfp4BatchItem* items, int count, int x_is_bf16, int out_kind, int M, int world, int rank,
                          void* const* peer_flags, int slot, const void* device_blob, void* host_blob) {
  if (!items || count < 1 || !device_blob || !host_blob || !aligned(device_blob, 256) || !aligned(host_blob, 8) ||
      !x_is_bf16 || world < 0 || world > dg::kMaxRanks || (world > 0 && (rank < 0 || rank >= world || !peer_flags)) ||
      slot < 0 || slot > 3)
    return (int)cudaErrorInvalidValue;
  DeviceState* st = device_state();
  if (!st) return (int)cudaErrorInvalidDevice;
  BatchHead head{};
  Params* out = reinterpret_cast<Params*>(static_cast<unsigned char*>(host_blob) + kBatchHead);
  int stage_bytes = 0, resident_bytes = 0, stages = 0;
  // One ring for all: the largest stage any GEMV needs, as many of them as fit. Behind the ring: room for one GEMV's
  // parameters (kernels without producer warps keep them there), then room for the largest resident activations
  // (every GEMV brings its own when its turn comes). If the resident ones cost the ring its third stage, once more
  // without them.
  for (int attempt = 0; attempt < 2; ++attempt) {
    stage_bytes = 0; resident_bytes = 0;
    for (int g = 0; g < count; ++g) {
      const DgNvfp4BatchItem& it = items[g];
      Params p{};
      if (!fill_nvfp4(p, it.x, it.ldx, x_is_bf16, it.codes, it.scales, it.blocked, it.inverse, out_kind, M, it.N, it.K))
        return (int)cudaErrorInvalidValue;
      if (world > 0) {
        if (!it.peer_out) return (int)cudaErrorInvalidValue;
        p.ldo = it.N;
        p.world = world; p.rank = rank; p.gather_slot = slot & 1; p.gather_nowait = slot >> 1;
        for (int q = 0; q < world; ++q) {
          if (!it.peer_out[q] || !peer_flags[q] || !aligned(peer_flags[q], 4)) return (int)cudaErrorInvalidValue;
          p.peer_out[q] = it.peer_out[q];
          p.peer_flag[q] = static_cast<unsigned int*>(peer_flags[q]);
        }
        p.out = it.peer_out[rank];
      } else {
        if (!it.out) return (int)cudaErrorInvalidValue;
        p.out = it.out; p.ldo = it.ldo;
      }
      int ctas = 0, smem = 0;
      // one grid for all: a CTA per SM, whatever a GEMV's size (a CTA without rows of a GEMV passes it by)
      if (const int code = prepare(dg::FMT_NVFP4, p, M, ctas, smem, st->sms * dg::ctas_per_sm(dg::FMT_NVFP4, M),
                                   attempt == 0))
        return code;
      if (p.stage_bytes > stage_bytes) stage_bytes = p.stage_bytes;
      if (p.x_resident) resident_bytes = std::max(resident_bytes, resident_bytes_of(dg::FMT_NVFP4, M, p.nblk));
      out[g] = p;
    }
    stages = (smem_limit(dg::FMT_NVFP4, M) - dg::kSmemHeader - (int)sizeof(Params) - resident_bytes) / stage_bytes;
    if (stages > dg::kMaxStages) stages = dg::kMaxStages;
    if (resident_bytes == 0 || stages >= 3) break;
  }
  if (stages < 2) return (int)cudaErrorInvalidValue;
  for (int g = 0; g < count; ++g) {
    out[g].stage_bytes = stage_bytes;
    out[g].stages = stages;
    out[g].x_res_off = dg::kSmemHeader + stages * stage_bytes + (int)sizeof(Params);
  }
  head.magic = kBatchMagic; head.count = count; head.M = M; head.ctas = st->sms * dg::ctas_per_sm(dg::FMT_NVFP4, M);
  head.smem = dg::kSmemHeader + stages * stage_bytes + (int)sizeof(Params) + resident_bytes;
  head.threads = 32 * (dg::consumer_warps(dg::FMT_NVFP4, M) + dg::producer_warps(dg::FMT_NVFP4, M));
  head.device_blob = device_blob;
  cudaGetDevice(&head.device);
  *reinterpret_cast<BatchHead*>(host_blob) = head;
  return 0;
}

int dg_enqueue_batch(const void* host_blob, void* stream) {
  if (!host_blob) return (int)cudaErrorInvalidValue;
  const BatchHead head = *reinterpret_cast<const BatchHead*>(host_blob);
  int device = -1;
  if (head.magic != kBatchMagic || head.count < 1 || head.M < 1 || head.M > DG_MAX_ROWS ||
      cudaGetDevice(&device) != cudaSuccess || device != head.device)
    return (int)cudaErrorInvalidValue;
  if (!device_state()) return (int)cudaErrorInvalidDevice;
  const Params* items = reinterpret_cast<const Params*>(static_cast<const unsigned char*>(head.device_blob) + kBatchHead);
  int count = head.count;
  void* args[] = {&items, &count};
  return launch_pdl(dg_batch_table_nvfp4_bf16[head.M - 1], args, head.ctas, head.threads, head.smem,
                    static_cast<cudaStream_t>(stream));
}

int dg_enqueue_fp8(const void* x, int ldx, int x_is_bf16, const uint8_t* codes, const float* row_scale,
                   const uint8_t* mx_scale, void* out, int ldo, int out_kind, int M, int N, int K, void* stream) {
  if (M < 1 || M > DG_MAX_ROWS || N < 1 || K < 16 || K % 16 || (mx_scale && K % 32) || (!row_scale == !mx_scale))
    return (int)cudaErrorInvalidValue;
  if (!x || !codes || !out || ldx % 8 || !aligned(x, 16) || !aligned(codes, 16) || !aligned(row_scale, 4) ||
      (out_kind != 0 && out_kind != 1))
    return (int)cudaErrorInvalidValue;
  Params p{};
  p.x = x; p.ldx = ldx; p.w = codes; p.scales = mx_scale; p.row_scale = row_scale; p.out = out; p.ldo = ldo;
  p.out_kind = out_kind == 0 ? dg::OUT_F32 : (x_is_bf16 ? dg::OUT_BF16 : dg::OUT_F16);
  p.N = N; p.K = K;
  p.scale_row_bytes = K / 32;
  p.scale_mode = !mx_scale ? dg::SCALES_NONE
                           : (K % 512 == 0 && aligned(mx_scale, 16)) ? dg::SCALES_STAGED : dg::SCALES_DIRECT;
  const int fmt = mx_scale ? dg::FMT_MXFP8 : dg::FMT_FP8;
  return launch((mx_scale ? 3 : 1) + (x_is_bf16 ? 0 : 1), fmt, p, M, static_cast<cudaStream_t>(stream));
}

int dg_enqueue_bf16(const void* x, int ldx, const void* w, void* out, int ldo, int out_kind, int M, int N, int K,
                    void* stream) {
  if (M < 1 || M > DG_MAX_ROWS || N < 1 || K < 8 || K % 8) return (int)cudaErrorInvalidValue;
  if (!x || !w || !out || ldx % 8 || !aligned(x, 16) || !aligned(w, 16) || (out_kind != 0 && out_kind != 1))
    return (int)cudaErrorInvalidValue;
  Params p{};
  p.x = x; p.ldx = ldx; p.w = static_cast<const uint8_t*>(w); p.out = out; p.ldo = ldo;
  p.out_kind = out_kind == 0 ? dg::OUT_F32 : dg::OUT_BF16;
  p.N = N; p.K = K;
  p.scale_mode = dg::SCALES_NONE;
  return launch(0, dg::FMT_BF16, p, M, static_cast<cudaStream_t>(stream));
}

int dg_hardware_decode(void) { return device_state() ? 1 : -1; }

int dg_plan(int fmt, int M, int N, int K, int plan[6]) {
  static const int kmult[4] = {8, 16, 32, 32};
  if (fmt < 0 || fmt > 3 || M < 1 || M > DG_MAX_ROWS || N < 1 || K < kmult[fmt] || K % kmult[fmt] || !plan)
    return (int)cudaErrorInvalidValue;
  int sms = 148;
  if (DeviceState* st = device_state()) sms = st->sms;
  Params p{};
  p.N = N; p.K = K;
  int ctas = 0, smem = 0;
  if (!make_plan(fmt, M, N, K, sms, p, ctas, smem)) return (int)cudaErrorInvalidValue;
  plan[0] = ctas; plan[1] = p.rows_per_warp; plan[2] = p.steps; plan[3] = p.stages; plan[4] = p.stage_bytes;
  plan[5] = smem;
  return 0;
}

int dg_take_status(void) {
  DeviceState* st = device_state();
  if (!st) return -(int)cudaErrorInvalidDevice;
  int word = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(&word, st->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && word) e = cudaMemset(st->status, 0, sizeof(int));
  return e == cudaSuccess ? word : -(int)e;
}

int dg_reset_noalloc_channel(int channel, void* stream) {
  if (channel < 0 || channel >= DG_NOALLOC_CHANNELS) return (int)cudaErrorInvalidValue;
  int current = 0;
  cudaError_t e = cudaGetDevice(&current);
  unsigned int* base = nullptr;
  if (e == cudaSuccess) e = gather_scratch_of(current, &base);
  if (e != cudaSuccess) return (int)e;
  return dg_reset_counters(base + 4 * channel, stream);
}

unsigned long long dg_set_wait_limit_ns(unsigned long long limit_ns) {
  return g_wait_limit_ns.exchange(limit_ns ? limit_ns : dg::kWaitLimitNs, std::memory_order_relaxed);
}

int dg_set_static_weights(int enabled) {
  return g_static_weights.exchange(enabled ? 1 : 0, std::memory_order_relaxed);
}

int dg_set_trace(void* buffer, int launches) {
  g_trace_base.store(nullptr, std::memory_order_release);
  g_trace_next.store(0, std::memory_order_relaxed);
  g_trace_capacity.store(buffer && launches > 0 ? launches : 0, std::memory_order_relaxed);
  if (buffer && launches > 0) g_trace_base.store(static_cast<unsigned long long*>(buffer), std::memory_order_release);
  return 0;
}

int dg_version(void) { return 102; }

}  // extern "C"
