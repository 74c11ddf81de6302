// Host-side plumbing shared by the translation units of libb200q.so.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

namespace b200q {

// Thread-local error text returned by b200q_last_error().
void set_error(const char* fmt, ...);

#define B200Q_CHECK_CUDA(expr)                                                              \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess) {                                                                \
      ::b200q::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return 1;                                                                             \
    }                                                                                       \
  } while (0)

#define B200Q_REQUIRE(cond, ...)        \
  do {                                  \
    if (!(cond)) {                      \
      ::b200q::set_error(__VA_ARGS__);  \
      return 2;                         \
    }                                   \
  } while (0)

// Bits of the device status word (b200q_status_word).  A kernel sets a bit and
// returns instead of trapping or spinning for ever; the host reads the word
// after synchronising.
enum StatusBits : uint32_t {
  STATUS_TMA_WAIT_TIMEOUT = 1u << 0,   // producer gave up waiting for a free pipeline slot
  STATUS_MMA_WAIT_TIMEOUT = 1u << 1,   // MMA issuer gave up waiting for operands or a free accumulator
  STATUS_EPI_WAIT_TIMEOUT = 1u << 2,   // epilogue gave up waiting for an accumulator
  STATUS_BAD_TMEM_ALLOC = 1u << 3,     // tensor-memory allocation returned an unexpected address
  STATUS_QUANT_WAIT_TIMEOUT = 1u << 4, // the staged quantize kernel gave up waiting for a row chunk or a free slot
  STATUS_BAD_INDEX = 1u << 5,          // an embedding lookup met a token outside its table (the row is zero)
  STATUS_SDPA_WAIT_TIMEOUT = 1u << 7,  // the tensor-core attention kernel gave up waiting for its MMAs
  STATUS_SELFTEST_WAIT_TIMEOUT = 1u << 6, // b200q_selftest_bounded_wait: the wait on a barrier nothing signals gave up, as it must
};

// Kernel families timed separately when profiling is on (b200q_profile_*).
enum KernelKind : int { KK_QUANT_TOKEN = 0, KK_DEQUANT_TOKEN, KK_QUANT_STATIC, KK_DEQUANT_STATIC, KK_WEIGHTS, KK_GEMM_UMMA,
                        KK_GEMM_SIMT, KK_EPILOGUE, KK_EMBEDDING, KK_LAYERNORM, KK_SDPA, KK_ADD, KK_COUNT };
constexpr int PROFILE_RING = 256;
constexpr int HOST_CHUNKS = 16;   // most pieces a host-buffer call is split into

struct HostStager;
constexpr int HOST_SLOTS = 3;   // row blocks of the page-locked staging ring per direction

struct Workspace {
  void* ptr = nullptr;
  size_t bytes = 0;
};

}  // namespace b200q

// The context behind the opaque handle of the C ABI: one per GPU, not thread safe.
struct b200q_ctx {
  int device = 0;
  int sm_count = 0;
  int l2_bytes = 0;
  cudaStream_t stream = nullptr;
  // copy streams and events of the pipelined host-buffer entry points (created on first use)
  cudaStream_t stream_h2d = nullptr, stream_d2h = nullptr;
  cudaEvent_t ev_in[b200q::HOST_CHUNKS] = {}, ev_done[b200q::HOST_CHUNKS] = {}, ev_free = nullptr;
  // pageable host buffers: a page-locked ring of HOST_SLOTS row blocks per direction and the threads that fill / drain it
  cudaEvent_t ev_out[b200q::HOST_CHUNKS] = {};
  void* pin_in = nullptr;
  void* pin_out = nullptr;
  size_t pin_in_bytes = 0, pin_out_bytes = 0;
  b200q::HostStager* stager = nullptr;
  int host_threads = 0;                  // threads of the stager (0: chosen at first use)
  // b200q_linear_f32_many: the stream the quantize of the next batch runs on, and the events between the two streams
  cudaStream_t stream_side = nullptr;
  cudaEvent_t ev_codes[2] = {}, ev_used[2] = {}, ev_entry = nullptr;
  cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
  uint32_t* status_dev = nullptr;        // device status word
  b200q::Workspace ws_q;                 // int8 activations of the fused linear
  b200q::Workspace ws_scales;            // their per-token scales
  b200q::Workspace ws_acc;               // int32 / f32 intermediates of the unfused paths
  b200q::Workspace ws_stage_in, ws_stage_out;  // device staging of the host-buffer entry points
  b200q::Workspace ws_range;             // row-range keys of the two-step per-token requantization (2 words per row)
  int requant_variant = 0;               // 0: ranges published by the GEMM epilogue + one-pass encode; 1: f32 result + full per-token quantize
  double wait_limit_s = 2.0;             // bound of every device-side wait
  int gemm_variant = 0;                  // 0 auto, 1 CUDA-core kernel only, 2 tensor cores with one CTA per tile, 3 with CTA pairs
  int tile_group = -1;                   // tensor-core GEMM: row blocks per group of the tile walking order (-1 chosen by size, 0 row block by row block)
  int epilogue_warps = 0;                // tensor-core GEMM, f32 output: 0 = sixteen epilogue warps for the exact sigmoid tails at K <= 1024, eight otherwise; 8 / 16 = always that many
  int quant_variant = 0;                 // 0 auto (rows staged in shared memory when they fit), 1 unstaged kernel only, 2 staged with both passes from shared memory
  uint32_t quant_staged_ready = 0;        // instances of the staged quantize kernel whose shared-memory attribute is set
  bool sdpa_ready = false;               // the attention kernels' shared-memory sizes have been raised
  bool sdpa_umma_ready = false;          // ... and that of the tensor-core attention kernel
  int tail_mode = 0;                     // 0: exact sigmoid tails; 1: hardware exp / reciprocal for f32 outputs (tolerance only)
  int sdpa_variant = 0;                  // 0: tcgen05 with three-way tf32 products when the shape allows; 1: mma.sync, three-way tf32; 2: tcgen05 or fail; 3: CUDA-core binary32 FMA
  uint64_t umma_ready_mask = 0;          // tensor-core kernel variants whose shared-memory attribute is set on this device
  uint64_t launches = 0;                 // kernels launched through this context
  bool capturing = false;                // between b200q_graph_begin and _end: calls are recorded, nothing may allocate or synchronise
  uint64_t capture_launches0 = 0;        // `launches` when the capture began
  // per-kernel CUDA-event timing (off by default): a ring of event pairs, folded into the sums when it wraps or is read
  bool profiling = false;
  cudaEvent_t prof_ev[b200q::PROFILE_RING][2] = {};
  int prof_kind[b200q::PROFILE_RING] = {};
  int prof_used = 0;
  double prof_ms[b200q::KK_COUNT] = {};
  uint64_t prof_n[b200q::KK_COUNT] = {};
};

namespace b200q {
int ws_reserve(b200q_ctx* ctx, Workspace& ws, size_t bytes);
int prof_fold(b200q_ctx* ctx);

// Brackets the kernel launches of one launcher with an event pair when profiling is on.
struct ProfScope {
  b200q_ctx* ctx;
  int idx = -1;
  ProfScope(b200q_ctx* c, int kind) : ctx(c) {
    if (!c->profiling) return;
    if (c->prof_used == PROFILE_RING) prof_fold(c);
    idx = c->prof_used++;
    c->prof_kind[idx] = kind;
    cudaEventRecord(c->prof_ev[idx][0], c->stream);
  }
  ~ProfScope() {
    if (idx >= 0) cudaEventRecord(ctx->prof_ev[idx][1], ctx->stream);
  }
};
}
