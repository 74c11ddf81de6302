// The C ABI of libb200q.so (declared in include/b200q.h): argument checks on the
// host before any launch, CUDA errors turned into return codes and a
// thread-local message, no exceptions or aborts across the boundary.
#include <cmath>
#include <cstdarg>
#include <cstring>
#include <new>
#include <thread>

#include "../../include/b200q.h"
#include <limits>
#include "common.cuh"
#include "kernels.cuh"

namespace b200q {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int ws_reserve(b200q_ctx* ctx, Workspace& ws, size_t bytes) {
  if (bytes <= ws.bytes) return 0;
  B200Q_REQUIRE(!ctx->capturing, "a workspace would have to grow while calls are being recorded: run the same calls once before b200q_graph_begin");
  // Stream-ordered, so a buffer still read by queued kernels is released after them.
  if (ws.ptr) B200Q_CHECK_CUDA(cudaFreeAsync(ws.ptr, ctx->stream));
  ws.ptr = nullptr;
  ws.bytes = 0;
  size_t want = bytes + bytes / 8;
  want = (want + 255) & ~size_t(255);
  B200Q_CHECK_CUDA(cudaMallocAsync(&ws.ptr, want, ctx->stream));
  ws.bytes = want;
  return 0;
}

int prof_fold(b200q_ctx* ctx) {
  for (int i = 0; i < ctx->prof_used; i++) {
    float ms = 0.0f;
    B200Q_CHECK_CUDA(cudaEventSynchronize(ctx->prof_ev[i][1]));
    B200Q_CHECK_CUDA(cudaEventElapsedTime(&ms, ctx->prof_ev[i][0], ctx->prof_ev[i][1]));
    ctx->prof_ms[ctx->prof_kind[i]] += ms;
    ctx->prof_n[ctx->prof_kind[i]] += 1;
  }
  ctx->prof_used = 0;
  return 0;
}

static int use_device(b200q_ctx* ctx) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_CHECK_CUDA(cudaSetDevice(ctx->device));
  return 0;
}

// Entry points that wait on the host or touch host memory cannot be part of a recorded sequence.
#define B200Q_NOT_CAPTURING(ctx, who) \
  B200Q_REQUIRE(!(ctx)->capturing, "%s is not allowed between b200q_graph_begin and b200q_graph_end", who)

static bool use_umma(b200q_ctx* ctx, const void* A, const void* W, int64_t M, int64_t N, int64_t K) {
  return ctx->gemm_variant != 1 && gemm_umma_supported(A, W, M, N, K);
}

#define B200Q_DIMS_OK(M, N, K)                                                                              \
  B200Q_REQUIRE((M) >= 0 && (N) >= 0 && (K) >= 0, "negative dimension (M=%lld N=%lld K=%lld)", (long long)(M), \
                (long long)(N), (long long)(K))

// quantized_dot + tail, any shape: tensor cores when possible, otherwise the CUDA-core
// kernel into a workspace followed by the tail kernel.
int gemm_i32_any(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K, int zpA, int zpB, int32_t* C) {
  if (!use_umma(ctx, A, W_nk, M, N, K)) return launch_gemm_i8_simt(ctx, A, W_nk, M, N, K, zpA, zpB, C);
  if (zpA == 0 && zpB == 0) return launch_gemm_i8_umma(ctx, A, W_nk, M, N, K, nullptr, nullptr, nullptr, 0, nullptr, C, nullptr, 1.0);
  // zero-points: the plain product on the tensor cores, then the three correction terms
  if (ws_reserve(ctx, ctx->ws_range, (size_t)(M + N) * sizeof(int32_t))) return 1;
  if (int e = launch_gemm_i8_umma(ctx, A, W_nk, M, N, K, nullptr, nullptr, nullptr, 0, nullptr, C, nullptr, 1.0)) return e;
  return launch_zero_point_fix(ctx, A, W_nk, M, N, K, zpA, zpB, (int32_t*)ctx->ws_range.ptr, C);
}

static int linear_core(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W, const float* w_scales,
                       const float* bias, int act, int64_t M, int64_t N, int64_t K, float* out_f32, int8_t* out_q,
                       double q_scale) {
  if (M == 0 || N == 0) return 0;
  if (K > 0 && use_umma(ctx, A, W, M, N, K))
    return launch_gemm_i8_umma(ctx, A, W, M, N, K, a_scales, w_scales, bias, act, out_f32, nullptr, out_q, q_scale);
  if (ws_reserve(ctx, ctx->ws_acc, (size_t)M * N * sizeof(int32_t))) return 1;
  int32_t* acc = (int32_t*)ctx->ws_acc.ptr;
  if (int e = launch_gemm_i8_simt(ctx, A, W, M, N, K, 0, 0, acc)) return e;
  return launch_epilogue(ctx, acc, M, N, a_scales, w_scales, bias, act, out_f32, out_q, q_scale);
}

// Linear followed by the per-token quantization of its result: y f32 [M,N] (scratch or a caller's buffer), codes with
// row stride ld_q, scales [M].  On the tensor-core path the range pass of that quantization happens in the GEMM's
// epilogue (every row's minimum and maximum are published as keys while the values are in registers) and a one-pass
// kernel then turns y into codes; otherwise y goes through the complete per-token quantize.  Same codes either way.
int linear_requant_token_core(b200q_ctx* ctx, const int8_t* A, const float* a_scales, int a_pieces, const int8_t* W,
                              const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K, float* y,
                              int8_t* out_q, int64_t ld_q, float* out_scales) {
  if (M == 0 || N == 0) return 0;
  const bool umma = K > 0 && use_umma(ctx, A, W, M, N, K);
  B200Q_REQUIRE(a_pieces == 1 || umma, "activations stored as column blocks need the tensor-core kernel (K %% 16 == 0, aligned operands)");
  if (umma && ctx->requant_variant == 0) {
    if (ws_reserve(ctx, ctx->ws_range, (size_t)2 * M * sizeof(uint32_t))) return 1;
    uint32_t* keys = (uint32_t*)ctx->ws_range.ptr;
    B200Q_CHECK_CUDA(cudaMemsetAsync(keys, 0, (size_t)2 * M * sizeof(uint32_t), ctx->stream));
    if (int e = launch_gemm_i8_umma(ctx, A, W, M, N, K, a_scales, w_scales, bias, act, y, nullptr, nullptr, 1.0, keys, a_pieces)) return e;
    return launch_quantize_rows_with_keys(ctx, y, M, N, N, keys, out_q, ld_q, out_scales, -127, 127);
  }
  if (umma) {
    if (int e = launch_gemm_i8_umma(ctx, A, W, M, N, K, a_scales, w_scales, bias, act, y, nullptr, nullptr, 1.0, nullptr, a_pieces)) return e;
  } else if (int e = linear_core(ctx, A, a_scales, W, w_scales, bias, act, M, N, K, y, nullptr, 1.0)) {
    return e;
  }
  if (ld_q == N) return launch_quantize_per_token(ctx, y, M, N, out_q, out_scales, -127, 127);
  // strided codes: range pass, then the encode that takes row strides
  if (ws_reserve(ctx, ctx->ws_range, (size_t)4 * M * sizeof(uint32_t))) return 1;
  float* mn = (float*)ctx->ws_range.ptr + 2 * M;
  float* mx = mn + M;
  if (int e = launch_row_range(ctx, y, M, N, N, mn, mx)) return e;
  return launch_quantize_rows_with_range(ctx, y, M, N, N, mn, mx, out_q, ld_q, out_scales, -127, 127);
}

}  // namespace b200q

using namespace b200q;

extern "C" {

int b200q_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    set_error("cudaGetDeviceCount failed: no usable CUDA driver or device");
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

const char* b200q_last_error(void) { return g_error; }

int b200q_create(int device, b200q_ctx** out) {
  B200Q_REQUIRE(out != nullptr, "b200q_create: null out pointer");
  *out = nullptr;
  int n = b200q_device_count();
  B200Q_REQUIRE(n > 0, "b200q_create: no CUDA device is available (this backend has no CPU fallback)");
  B200Q_REQUIRE(device >= 0 && device < n, "b200q_create: device %d out of range (0..%d)", device, n - 1);
  B200Q_CHECK_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  B200Q_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
  B200Q_REQUIRE(prop.major == 10, "b200q_create: device %d is sm_%d%d; this library is built for sm_100a only", device,
                prop.major, prop.minor);
  b200q_ctx* ctx = new (std::nothrow) b200q_ctx();
  B200Q_REQUIRE(ctx != nullptr, "b200q_create: out of host memory");
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->l2_bytes = prop.l2CacheSize;
  cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev_start);
  if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev_stop);
  if (e == cudaSuccess) e = cudaMalloc(&ctx->status_dev, sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(ctx->status_dev, 0, sizeof(uint32_t));
  if (e != cudaSuccess) {
    set_error("b200q_create: %s", cudaGetErrorString(e));
    b200q_destroy(ctx);
    return 1;
  }
  // The fixed scratch of b200q_linear_f32_noalloc comes into being here (its module is loaded on this device), not
  // inside the first call of that entry point.
  if (int pe = noalloc_prepare(device)) {
    b200q_destroy(ctx);
    return pe;
  }
  *out = ctx;
  return 0;
}

void b200q_destroy(b200q_ctx* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  Workspace* all[] = {&ctx->ws_q, &ctx->ws_scales, &ctx->ws_acc, &ctx->ws_stage_in, &ctx->ws_stage_out, &ctx->ws_range};
  for (Workspace* w : all)
    if (w->ptr) cudaFree(w->ptr);
  if (ctx->status_dev) cudaFree(ctx->status_dev);
  for (int i = 0; i < PROFILE_RING; i++)
    for (int j = 0; j < 2; j++)
      if (ctx->prof_ev[i][j]) cudaEventDestroy(ctx->prof_ev[i][j]);
  for (int i = 0; i < HOST_CHUNKS; i++) {
    if (ctx->ev_in[i]) cudaEventDestroy(ctx->ev_in[i]);
    if (ctx->ev_done[i]) cudaEventDestroy(ctx->ev_done[i]);
    if (ctx->ev_out[i]) cudaEventDestroy(ctx->ev_out[i]);
  }
  for (int i = 0; i < 2; i++) {
    if (ctx->ev_codes[i]) cudaEventDestroy(ctx->ev_codes[i]);
    if (ctx->ev_used[i]) cudaEventDestroy(ctx->ev_used[i]);
  }
  if (ctx->ev_entry) cudaEventDestroy(ctx->ev_entry);
  if (ctx->stream_side) {
    cudaStreamSynchronize(ctx->stream_side);
    cudaStreamDestroy(ctx->stream_side);
  }
  host_stager_destroy(ctx->stager);
  if (ctx->pin_in) cudaFreeHost(ctx->pin_in);
  if (ctx->pin_out) cudaFreeHost(ctx->pin_out);
  if (ctx->ev_free) cudaEventDestroy(ctx->ev_free);
  if (ctx->stream_h2d) cudaStreamDestroy(ctx->stream_h2d);
  if (ctx->stream_d2h) cudaStreamDestroy(ctx->stream_d2h);
  if (ctx->ev_start) cudaEventDestroy(ctx->ev_start);
  if (ctx->ev_stop) cudaEventDestroy(ctx->ev_stop);
  if (ctx->stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
}

int b200q_sync(b200q_ctx* ctx) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_sync");
  B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  return 0;
}

int b200q_status_word(b200q_ctx* ctx, uint32_t* out) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_status_word");
  B200Q_REQUIRE(out != nullptr, "b200q_status_word: null out pointer");
  B200Q_CHECK_CUDA(cudaMemcpyAsync(out, ctx->status_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost, ctx->stream));
  B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  return 0;
}

int b200q_clear_status(b200q_ctx* ctx) {
  if (use_device(ctx)) return 1;
  B200Q_CHECK_CUDA(cudaMemsetAsync(ctx->status_dev, 0, sizeof(uint32_t), ctx->stream));
  return 0;
}

int b200q_set_wait_limit(b200q_ctx* ctx, double seconds) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(seconds > 0 && seconds <= 60, "b200q_set_wait_limit: %g s is outside (0, 60]", seconds);
  ctx->wait_limit_s = seconds;
  return 0;
}

int b200q_set_tail_mode(b200q_ctx* ctx, int mode) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(mode == 0 || mode == 1, "b200q_set_tail_mode: unknown mode %d", mode);
  ctx->tail_mode = mode;
  return 0;
}

int b200q_set_sdpa_variant(b200q_ctx* ctx, int variant) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(variant >= 0 && variant <= 3, "b200q_set_sdpa_variant: unknown variant %d", variant);
  ctx->sdpa_variant = variant;
  return 0;
}

int b200q_set_gemm_variant(b200q_ctx* ctx, int variant) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(variant >= 0 && variant <= 3, "b200q_set_gemm_variant: unknown variant %d", variant);
  ctx->gemm_variant = variant;
  return 0;
}

int b200q_set_tile_group(b200q_ctx* ctx, int row_blocks) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(row_blocks >= -1 && row_blocks <= 65536, "b200q_set_tile_group: %d is not -1, 0 or a group size", row_blocks);
  ctx->tile_group = row_blocks;
  return 0;
}

int b200q_set_host_threads(b200q_ctx* ctx, int threads) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(threads >= 0 && threads <= 64, "b200q_set_host_threads: %d is not between 0 and 64", threads);
  B200Q_REQUIRE(ctx->stager == nullptr, "b200q_set_host_threads: the staging threads of this context already run");
  ctx->host_threads = threads;
  return 0;
}

int b200q_set_epilogue_warps(b200q_ctx* ctx, int warps) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(warps == 0 || warps == 8 || warps == 16, "b200q_set_epilogue_warps: %d is not 0, 8 or 16", warps);
  ctx->epilogue_warps = warps;
  return 0;
}

int b200q_set_requant_variant(b200q_ctx* ctx, int variant) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(variant == 0 || variant == 1, "b200q_set_requant_variant: unknown variant %d", variant);
  ctx->requant_variant = variant;
  return 0;
}

int b200q_set_quant_variant(b200q_ctx* ctx, int variant) {
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_REQUIRE(variant >= 0 && variant <= 4, "b200q_set_quant_variant: unknown variant %d", variant);
  ctx->quant_variant = variant;
  return 0;
}

int b200q_profile_enable(b200q_ctx* ctx, int on) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_profile_enable");
  if (on && !ctx->prof_ev[0][0]) {
    for (int i = 0; i < PROFILE_RING; i++)
      for (int j = 0; j < 2; j++) B200Q_CHECK_CUDA(cudaEventCreate(&ctx->prof_ev[i][j]));
  }
  if (!on && ctx->profiling) prof_fold(ctx);
  ctx->profiling = on != 0;
  return 0;
}

int b200q_profile_reset(b200q_ctx* ctx) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_profile_reset");
  if (prof_fold(ctx)) return 1;
  for (int k = 0; k < KK_COUNT; k++) { ctx->prof_ms[k] = 0.0; ctx->prof_n[k] = 0; }
  return 0;
}

int b200q_profile_read(b200q_ctx* ctx, int kind, double* total_ms, uint64_t* launches) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_profile_read");
  B200Q_REQUIRE(kind >= 0 && kind < KK_COUNT, "b200q_profile_read: unknown kernel family %d", kind);
  B200Q_REQUIRE(total_ms && launches, "b200q_profile_read: null out pointer");
  if (prof_fold(ctx)) return 1;
  *total_ms = ctx->prof_ms[kind];
  *launches = ctx->prof_n[kind];
  return 0;
}

uint64_t b200q_launch_count(b200q_ctx* ctx) { return ctx ? ctx->launches : 0; }
int b200q_sm_count(b200q_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

// ---------------------------------------------------------------- memory
int b200q_alloc(b200q_ctx* ctx, size_t bytes, void** dev) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_alloc");
  B200Q_REQUIRE(dev != nullptr, "b200q_alloc: null out pointer");
  *dev = nullptr;
  if (bytes == 0) bytes = 16;
  B200Q_CHECK_CUDA(cudaMalloc(dev, bytes));
  return 0;
}

int b200q_free(b200q_ctx* ctx, void* dev) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_free");
  if (!dev) return 0;
  B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  B200Q_CHECK_CUDA(cudaFree(dev));
  return 0;
}

int b200q_memset(b200q_ctx* ctx, void* dev, int byte_value, size_t bytes) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(dev != nullptr || bytes == 0, "b200q_memset: null pointer");
  if (bytes) B200Q_CHECK_CUDA(cudaMemsetAsync(dev, byte_value, bytes, ctx->stream));
  return 0;
}

int b200q_upload(b200q_ctx* ctx, void* dev, const void* host, size_t bytes) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_upload");
  B200Q_REQUIRE((dev && host) || bytes == 0, "b200q_upload: null pointer");
  if (bytes) {
    B200Q_CHECK_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  return 0;
}

int b200q_download(b200q_ctx* ctx, void* host, const void* dev, size_t bytes) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_download");
  B200Q_REQUIRE((dev && host) || bytes == 0, "b200q_download: null pointer");
  if (bytes) {
    B200Q_CHECK_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  }
  return 0;
}

int b200q_host_alloc(b200q_ctx* ctx, size_t bytes, void** host) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(host != nullptr, "b200q_host_alloc: null out pointer");
  *host = nullptr;
  if (bytes == 0) bytes = 16;
  B200Q_CHECK_CUDA(cudaMallocHost(host, bytes));
  return 0;
}

int b200q_host_free(b200q_ctx* ctx, void* host) {
  if (use_device(ctx)) return 1;
  if (host) B200Q_CHECK_CUDA(cudaFreeHost(host));
  return 0;
}

int b200q_host_register(b200q_ctx* ctx, void* host, size_t bytes) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(host != nullptr && bytes > 0, "b200q_host_register: null pointer or empty range");
  const cudaError_t e = cudaHostRegister(host, bytes, cudaHostRegisterDefault);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();   // a refused registration is the caller's to handle: it must not show up in a later launch check
    set_error("b200q_host_register: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

int b200q_host_unregister(b200q_ctx* ctx, void* host) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(host != nullptr, "b200q_host_unregister: null pointer");
  const cudaError_t e = cudaHostUnregister(host);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    set_error("b200q_host_unregister: %s", cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

// ---------------------------------------------------------------- timing
int b200q_timer_start(b200q_ctx* ctx) {
  if (use_device(ctx)) return 1;
  B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_start, ctx->stream));
  return 0;
}

int b200q_timer_stop(b200q_ctx* ctx, float* elapsed_ms) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_timer_stop");
  B200Q_REQUIRE(elapsed_ms != nullptr, "b200q_timer_stop: null out pointer");
  B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_stop, ctx->stream));
  B200Q_CHECK_CUDA(cudaEventSynchronize(ctx->ev_stop));
  B200Q_CHECK_CUDA(cudaEventElapsedTime(elapsed_ms, ctx->ev_start, ctx->ev_stop));
  return 0;
}

// ---------------------------------------------------------------- ops
int b200q_quantize_per_token(b200q_ctx* ctx, const float* x, int64_t M, int64_t K, int8_t* q, float* scales, int qmin,
                             int qmax) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(M, 0, K);
  B200Q_REQUIRE(M == 0 || K == 0 || (x && q), "b200q_quantize_per_token: null data pointer");
  B200Q_REQUIRE(M == 0 || scales, "b200q_quantize_per_token: null scales pointer");
  B200Q_REQUIRE(qmin >= -128 && qmax <= 127 && qmin < qmax, "b200q_quantize_per_token: clamp [%d,%d] is not an int8 range", qmin,
                qmax);
  B200Q_REQUIRE(K > 0 || M == 0, "b200q_quantize_per_token: rows of zero length have no range");
  return launch_quantize_per_token(ctx, x, M, K, q, scales, qmin, qmax);
}

int b200q_dequantize_per_token(b200q_ctx* ctx, const int8_t* q, const float* scales, int64_t M, int64_t K, float* y) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(M, 0, K);
  B200Q_REQUIRE(M == 0 || K == 0 || (q && scales && y), "b200q_dequantize_per_token: null pointer");
  return launch_dequantize_per_token(ctx, q, scales, M, K, y);
}

int b200q_row_range(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld, float* row_min, float* row_max) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(M, N, 0);
  B200Q_REQUIRE(ld >= N, "b200q_row_range: row stride %lld is smaller than the row length %lld", (long long)ld, (long long)N);
  B200Q_REQUIRE(M == 0 || (row_min && row_max && (y || N == 0)), "b200q_row_range: null pointer");
  return launch_row_range(ctx, y, M, N, ld, row_min, row_max);
}

int b200q_quantize_rows_with_range(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld_in, const float* row_min,
                                   const float* row_max, int8_t* q, int64_t ld_out, float* scales, int qmin, int qmax) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(M, N, 0);
  B200Q_REQUIRE(ld_in >= N && ld_out >= N, "b200q_quantize_rows_with_range: a row stride is smaller than the row length");
  B200Q_REQUIRE(M == 0 || N == 0 || (y && q && row_min && row_max), "b200q_quantize_rows_with_range: null pointer");
  B200Q_REQUIRE(qmin >= -128 && qmax <= 127 && qmin < qmax, "b200q_quantize_rows_with_range: clamp [%d,%d] is not an int8 range", qmin, qmax);
  return launch_quantize_rows_with_range(ctx, y, M, N, ld_in, row_min, row_max, q, ld_out, scales, qmin, qmax);
}

int b200q_quantize_static(b200q_ctx* ctx, const float* x, int64_t n, double scale, int zero_point, int dst_kind, void* q) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(n >= 0, "b200q_quantize_static: negative length");
  B200Q_REQUIRE(n == 0 || (x && q), "b200q_quantize_static: null pointer");
  B200Q_REQUIRE(dst_kind == B200Q_I8 || dst_kind == B200Q_UI8, "b200q_quantize_static: target must be int8 or uint8");
  B200Q_REQUIRE(scale == scale && scale != 0.0, "b200q_quantize_static: scale must be a non-zero number");
  B200Q_REQUIRE(zero_point >= -128 && zero_point <= 255, "b200q_quantize_static: zero point %d outside 8-bit range", zero_point);
  return launch_quantize_static(ctx, x, n, scale, zero_point, dst_kind, q);
}

int b200q_dequantize_static(b200q_ctx* ctx, const void* q, int src_kind, int64_t n, double scale, int zero_point, float* y) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(n >= 0, "b200q_dequantize_static: negative length");
  B200Q_REQUIRE(n == 0 || (q && y), "b200q_dequantize_static: null pointer");
  B200Q_REQUIRE(src_kind == B200Q_I8 || src_kind == B200Q_UI8 || src_kind == B200Q_I32,
                "b200q_dequantize_static: source must be int8, uint8 or int32");
  return launch_dequantize_static(ctx, q, src_kind, n, scale, zero_point, y);
}

int b200q_quantize_weights_per_channel(b200q_ctx* ctx, const float* w, int64_t N, int64_t K, int layout, int8_t* qw,
                                       float* w_scales32, double* w_scales64) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(0, N, K);
  B200Q_REQUIRE(layout == B200Q_W_NK || layout == B200Q_W_KN, "b200q_quantize_weights_per_channel: unknown layout %d", layout);
  B200Q_REQUIRE(N == 0 || K == 0 || (w && qw), "b200q_quantize_weights_per_channel: null pointer");
  // per_channel scheme: clampRange() is [-128,127] (quantization_types.ts:62-73)
  return launch_quantize_weights(ctx, w, N, K, layout, -128, 127, qw, w_scales32, w_scales64);
}

int b200q_transpose_i8(b200q_ctx* ctx, const int8_t* w_kn, int64_t K, int64_t N, int8_t* w_nk) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(0, N, K);
  B200Q_REQUIRE(N == 0 || K == 0 || (w_kn && w_nk), "b200q_transpose_i8: null pointer");
  return launch_transpose_i8(ctx, w_kn, K, N, w_nk);
}

int b200q_int8_gemm_i32(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K, int zpA, int zpW,
                        int32_t* C) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(M, N, K);
  B200Q_REQUIRE(M == 0 || N == 0 || C, "b200q_int8_gemm_i32: null output");
  B200Q_REQUIRE(M == 0 || N == 0 || K == 0 || (A && W_nk), "b200q_int8_gemm_i32: null operand");
  B200Q_REQUIRE(zpA >= -128 && zpA <= 127 && zpW >= -128 && zpW <= 127, "b200q_int8_gemm_i32: zero point outside int8");
  if (M == 0 || N == 0) return 0;
  if (K == 0) {
    B200Q_CHECK_CUDA(cudaMemsetAsync(C, 0, (size_t)M * N * sizeof(int32_t), ctx->stream));
    return 0;
  }
  return gemm_i32_any(ctx, A, W_nk, M, N, K, zpA, zpW, C);
}

int b200q_quantize_per_group(b200q_ctx* ctx, const float* x, int64_t n, int64_t group_size, int num_bits, int8_t* q,
                             double* scales64, float* scales32) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(n >= 0 && group_size >= 1, "b200q_quantize_per_group: bad size (n=%lld group_size=%lld)", (long long)n,
                (long long)group_size);
  B200Q_REQUIRE(num_bits >= 2 && num_bits <= 8, "b200q_quantize_per_group: %d bits do not fit an int8 code", num_bits);
  B200Q_REQUIRE(n == 0 || x, "b200q_quantize_per_group: null input");
  return launch_quantize_per_group(ctx, x, n, group_size, num_bits, q, scales64, scales32);
}

int b200q_dequantize_per_group(b200q_ctx* ctx, const int8_t* q, int64_t n, int64_t group_size, const double* scales64,
                               double* y64, float* y32) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(n >= 0 && group_size >= 1, "b200q_dequantize_per_group: bad size (n=%lld group_size=%lld)", (long long)n,
                (long long)group_size);
  B200Q_REQUIRE(n == 0 || (q && scales64), "b200q_dequantize_per_group: null codes or scales");
  return launch_dequantize_per_group(ctx, q, n, group_size, scales64, y64, y32);
}

int b200q_quantized_conv2d(b200q_ctx* ctx, const int8_t* in, const int8_t* ker, int64_t N, int64_t C, int64_t H, int64_t W,
                           int64_t O, int64_t KH, int64_t KW, int stride_h, int stride_w, int pad_top, int pad_bottom,
                           int pad_left, int pad_right, int dil_h, int dil_w, int groups, int zp_in, int zp_ker, int layout,
                           int32_t* out) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_quantized_conv2d");
  B200Q_REQUIRE(N >= 0 && C >= 1 && H >= 1 && W >= 1 && O >= 0 && KH >= 1 && KW >= 1,
                "b200q_quantized_conv2d: bad extent (N=%lld C=%lld H=%lld W=%lld O=%lld KH=%lld KW=%lld)", (long long)N, (long long)C,
                (long long)H, (long long)W, (long long)O, (long long)KH, (long long)KW);
  B200Q_REQUIRE(stride_h >= 1 && stride_w >= 1 && dil_h >= 1 && dil_w >= 1, "b200q_quantized_conv2d: strides and dilations start at 1");
  B200Q_REQUIRE(pad_top >= 0 && pad_bottom >= 0 && pad_left >= 0 && pad_right >= 0, "b200q_quantized_conv2d: negative padding");
  B200Q_REQUIRE(groups >= 1 && C % groups == 0 && O % groups == 0,
                "b200q_quantized_conv2d: %d groups do not divide C=%lld and O=%lld", groups, (long long)C, (long long)O);
  B200Q_REQUIRE(zp_in >= -128 && zp_in <= 127 && zp_ker >= -128 && zp_ker <= 127, "b200q_quantized_conv2d: zero point outside int8");
  B200Q_REQUIRE(layout == B200Q_CONV_NCHW || layout == B200Q_CONV_NHWC, "b200q_quantized_conv2d: unknown layout %d", layout);
  B200Q_REQUIRE(H + pad_top + pad_bottom >= (KH - 1) * dil_h + 1 && W + pad_left + pad_right >= (KW - 1) * dil_w + 1,
                "b200q_quantized_conv2d: the dilated kernel is larger than the padded input");
  B200Q_REQUIRE(N <= 65535, "b200q_quantized_conv2d: at most 65535 images per call");
  B200Q_REQUIRE((C / groups) * KH * KW <= 131072, "b200q_quantized_conv2d: more than 131072 taps per output could overflow the int32 sum");
  if (N == 0 || O == 0) return 0;
  B200Q_REQUIRE(in && ker && out, "b200q_quantized_conv2d: null pointer");
  return launch_quantized_conv2d(ctx, in, ker, N, C, H, W, O, KH, KW, stride_h, stride_w, pad_top, pad_bottom, pad_left, pad_right,
                                 dil_h, dil_w, groups, zp_in, zp_ker, layout, out);
}

int b200q_shift_u8_to_i8(b200q_ctx* ctx, const uint8_t* src, int64_t n, int8_t* dst) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(n >= 0 && (n == 0 || (src && dst)), "b200q_shift_u8_to_i8: bad length or null pointer");
  return launch_shift_u8_i8(ctx, src, n, dst);
}

int b200q_epilogue(b200q_ctx* ctx, const int32_t* acc, int64_t M, int64_t N, const float* a_scales, const float* w_scales,
                   const float* bias, int act, float* out) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(M, N, 0);
  B200Q_REQUIRE(M == 0 || N == 0 || (acc && w_scales && out), "b200q_epilogue: null pointer");
  B200Q_REQUIRE(act >= 0 && act <= 4, "b200q_epilogue: unknown activation %d", act);
  return launch_epilogue(ctx, acc, M, N, a_scales, w_scales, bias, act, out, nullptr, 1.0);
}

int b200q_epilogue_tensor_scale(b200q_ctx* ctx, const int32_t* acc, int64_t M, int64_t N, double scale, const float* bias, int act,
                                float* out) {
  if (use_device(ctx)) return 1;
  B200Q_DIMS_OK(M, N, 0);
  B200Q_REQUIRE(M == 0 || N == 0 || (acc && out), "b200q_epilogue_tensor_scale: null pointer");
  B200Q_REQUIRE(act >= 0 && act <= 4, "b200q_epilogue_tensor_scale: unknown activation %d", act);
  return launch_epilogue(ctx, acc, M, N, nullptr, nullptr, bias, act, out, nullptr, 1.0, scale);
}

static int check_linear(const char* who, const void* A, const void* W, const float* w_scales, int act, int64_t M, int64_t N,
                        int64_t K, const void* out) {
  B200Q_DIMS_OK(M, N, K);
  B200Q_REQUIRE(act >= 0 && act <= 4, "%s: unknown activation %d", who, act);
  B200Q_REQUIRE(M == 0 || N == 0 || (out && w_scales), "%s: null output or weight scales", who);
  B200Q_REQUIRE(M == 0 || N == 0 || K == 0 || (A && W), "%s: null operand", who);
  return 0;
}

int b200q_int8_linear(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W_nk, const float* w_scales,
                      const float* bias, int act, int64_t M, int64_t N, int64_t K, float* out) {
  if (use_device(ctx)) return 1;
  if (int e = check_linear("b200q_int8_linear", A, W_nk, w_scales, act, M, N, K, out)) return e;
  return linear_core(ctx, A, a_scales, W_nk, w_scales, bias, act, M, N, K, out, nullptr, 1.0);
}

int b200q_int8_linear_gathered(b200q_ctx* ctx, const int8_t* A, const float* a_scales, int a_blocks, const int8_t* W_nk,
                               const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K, float* out) {
  if (use_device(ctx)) return 1;
  if (int e = check_linear("b200q_int8_linear_gathered", A, W_nk, w_scales, act, M, N, K, out)) return e;
  B200Q_REQUIRE(a_blocks >= 1, "b200q_int8_linear_gathered: %d column blocks", a_blocks);
  if (M == 0 || N == 0) return 0;
  B200Q_REQUIRE(K > 0 && use_umma(ctx, A, W_nk, M, N, K),
                "b200q_int8_linear_gathered: needs the tensor-core kernel (K %% 16 == 0, 16-byte aligned operands)");
  return launch_gemm_i8_umma(ctx, A, W_nk, M, N, K, a_scales, w_scales, bias, act, out, nullptr, nullptr, 1.0, nullptr, a_blocks);
}

int b200q_int8_linear_requant_static(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W_nk,
                                     const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K,
                                     double out_scale, int8_t* out_q) {
  if (use_device(ctx)) return 1;
  if (int e = check_linear("b200q_int8_linear_requant_static", A, W_nk, w_scales, act, M, N, K, out_q)) return e;
  B200Q_REQUIRE(out_scale == out_scale && out_scale != 0.0, "b200q_int8_linear_requant_static: scale must be a non-zero number");
  return linear_core(ctx, A, a_scales, W_nk, w_scales, bias, act, M, N, K, nullptr, out_q, out_scale);
}

int b200q_int8_linear_requant_token(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W_nk,
                                    const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K,
                                    int8_t* out_q, float* out_scales) {
  if (use_device(ctx)) return 1;
  if (int e = check_linear("b200q_int8_linear_requant_token", A, W_nk, w_scales, act, M, N, K, out_q)) return e;
  B200Q_REQUIRE(M == 0 || out_scales, "b200q_int8_linear_requant_token: null scales output");
  if (M == 0 || N == 0) return 0;
  // The f32 result lives in its own workspace: ws_acc may be in use by the CUDA-core path.
  if (ws_reserve(ctx, ctx->ws_stage_out, (size_t)M * N * sizeof(float))) return 1;
  float* y = (float*)ctx->ws_stage_out.ptr;
  return linear_requant_token_core(ctx, A, a_scales, 1, W_nk, w_scales, bias, act, M, N, K, y, out_q, N, out_scales);
}

int b200q_int8_linear_f32_requant_token(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W_nk,
                                        const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K,
                                        float* out_f32, int8_t* out_q, float* out_scales) {
  if (use_device(ctx)) return 1;
  if (int e = check_linear("b200q_int8_linear_f32_requant_token", A, W_nk, w_scales, act, M, N, K, out_q)) return e;
  B200Q_REQUIRE(M == 0 || N == 0 || (out_scales && out_f32), "b200q_int8_linear_f32_requant_token: null output");
  if (M == 0 || N == 0) return 0;
  return linear_requant_token_core(ctx, A, a_scales, 1, W_nk, w_scales, bias, act, M, N, K, out_f32, out_q, N, out_scales);
}

int b200q_linear_f32(b200q_ctx* ctx, const float* x, const int8_t* W_nk, const float* w_scales, const float* bias, int act,
                     int64_t M, int64_t N, int64_t K, float* out) {
  if (use_device(ctx)) return 1;
  if (int e = check_linear("b200q_linear_f32", x, W_nk, w_scales, act, M, N, K, out)) return e;
  B200Q_REQUIRE(K > 0 || M == 0, "b200q_linear_f32: rows of zero length have no range");
  if (M == 0 || N == 0) return 0;
  if (ws_reserve(ctx, ctx->ws_q, (size_t)M * K)) return 1;
  if (ws_reserve(ctx, ctx->ws_scales, (size_t)M * sizeof(float))) return 1;
  int8_t* q = (int8_t*)ctx->ws_q.ptr;
  float* s = (float*)ctx->ws_scales.ptr;
  if (int e = launch_quantize_per_token(ctx, x, M, K, q, s, -127, 127)) return e;
  return linear_core(ctx, q, s, W_nk, w_scales, bias, act, M, N, K, out, nullptr, 1.0);
}

// Independent batches through the same linear, as a serving loop has them queued: the per-token quantize of batch i+1
// runs on a second stream while the GEMM of batch i holds the tensor cores -- the quantize is bound by HBM, the GEMM is
// not, and a quantize block fits beside the GEMM's one CTA per SM.  Two sets of codes and scales alternate; events order
// quantize i before GEMM i and GEMM i before quantize i+2 (which reuses its codes).  Every batch gets the result of
// b200q_linear_f32.  Stream-ordered like every other call: the work before it on the context's stream is waited for
// (once, at entry), the work after it sees all results.
int b200q_linear_f32_many(b200q_ctx* ctx, int count, const float* const* x, const int8_t* W_nk, const float* w_scales,
                          const float* bias, int act, int64_t M, int64_t N, int64_t K, float* const* out) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_linear_f32_many");
  B200Q_REQUIRE(count >= 0, "b200q_linear_f32_many: negative batch count");
  B200Q_REQUIRE(count == 0 || (x && out), "b200q_linear_f32_many: null array of batches");
  for (int i = 0; i < count; i++)
    if (int e = check_linear("b200q_linear_f32_many", x[i], W_nk, w_scales, act, M, N, K, out[i])) return e;
  B200Q_REQUIRE(K > 0 || M == 0, "b200q_linear_f32_many: rows of zero length have no range");
  if (count == 0 || M == 0 || N == 0) return 0;
  if (count == 1) return b200q_linear_f32(ctx, x[0], W_nk, w_scales, bias, act, M, N, K, out[0]);
  if (!ctx->stream_side) {
    B200Q_CHECK_CUDA(cudaStreamCreateWithFlags(&ctx->stream_side, cudaStreamNonBlocking));
    for (int i = 0; i < 2; i++) {
      B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&ctx->ev_codes[i], cudaEventDisableTiming));
      B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&ctx->ev_used[i], cudaEventDisableTiming));
    }
    B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&ctx->ev_entry, cudaEventDisableTiming));
  }
  const size_t codes = ((size_t)M * K + 255) & ~size_t(255);
  if (ws_reserve(ctx, ctx->ws_q, 2 * codes)) return 1;
  if (ws_reserve(ctx, ctx->ws_scales, (size_t)2 * M * sizeof(float))) return 1;
  // the second stream starts after everything queued so far (the inputs' producers, the workspaces' allocation)
  B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_entry, ctx->stream));
  B200Q_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream_side, ctx->ev_entry, 0));
  cudaStream_t main_stream = ctx->stream;
  for (int i = 0; i < count; i++) {
    const int slot = i & 1;
    int8_t* q = (int8_t*)ctx->ws_q.ptr + (size_t)slot * codes;
    float* sc = (float*)ctx->ws_scales.ptr + (size_t)slot * M;
    if (i >= 2) B200Q_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream_side, ctx->ev_used[slot], 0));
    ctx->stream = ctx->stream_side;                 // the launcher enqueues on the context's current stream
    const int qe = launch_quantize_per_token(ctx, x[i], M, K, q, sc, -127, 127);
    ctx->stream = main_stream;
    if (qe) return qe;
    B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_codes[slot], ctx->stream_side));
    B200Q_CHECK_CUDA(cudaStreamWaitEvent(main_stream, ctx->ev_codes[slot], 0));
    if (int e = linear_core(ctx, q, sc, W_nk, w_scales, bias, act, M, N, K, out[i], nullptr, 1.0)) return e;
    B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_used[slot], main_stream));
  }
  return 0;
}

// True when the copy engines can stream from / to the pointer directly: page-locked by cudaHostAlloc /
// cudaHostRegister, or managed.  Ordinary malloc'ed memory reports cudaMemoryTypeUnregistered.
static bool host_pointer_is_page_locked(const void* p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeHost || attr.type == cudaMemoryTypeManaged;
}

// The page-locked ring (HOST_SLOTS row blocks per direction that is staged) and the copy threads.
static int host_staging_ready(b200q_ctx* ctx, size_t in_block, size_t out_block) {
  if (!ctx->stager) {
    int n = ctx->host_threads;
    if (n <= 0) {
      const unsigned hw = std::thread::hardware_concurrency();
      n = hw >= 16 ? 8 : (hw >= 4 ? (int)hw / 2 : 1);
    }
    ctx->stager = host_stager_create(n);
    B200Q_REQUIRE(ctx->stager != nullptr, "out of host memory for the staging threads");
  }
  if (in_block * HOST_SLOTS > ctx->pin_in_bytes) {
    B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream_h2d));
    if (ctx->pin_in) B200Q_CHECK_CUDA(cudaFreeHost(ctx->pin_in));
    ctx->pin_in = nullptr;
    ctx->pin_in_bytes = 0;
    B200Q_CHECK_CUDA(cudaHostAlloc(&ctx->pin_in, in_block * HOST_SLOTS, cudaHostAllocDefault));
    ctx->pin_in_bytes = in_block * HOST_SLOTS;
  }
  if (out_block * HOST_SLOTS > ctx->pin_out_bytes) {
    B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream_d2h));
    if (ctx->pin_out) B200Q_CHECK_CUDA(cudaFreeHost(ctx->pin_out));
    ctx->pin_out = nullptr;
    ctx->pin_out_bytes = 0;
    B200Q_CHECK_CUDA(cudaHostAlloc(&ctx->pin_out, out_block * HOST_SLOTS, cudaHostAllocDefault));
    ctx->pin_out_bytes = out_block * HOST_SLOTS;
  }
  return 0;
}

static int host_pipeline_ready(b200q_ctx* ctx) {
  if (ctx->stream_h2d) return 0;
  B200Q_CHECK_CUDA(cudaStreamCreateWithFlags(&ctx->stream_h2d, cudaStreamNonBlocking));
  B200Q_CHECK_CUDA(cudaStreamCreateWithFlags(&ctx->stream_d2h, cudaStreamNonBlocking));
  for (int i = 0; i < HOST_CHUNKS; i++) {
    B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&ctx->ev_in[i], cudaEventDisableTiming));
    B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&ctx->ev_done[i], cudaEventDisableTiming));
    B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&ctx->ev_out[i], cudaEventDisableTiming));
  }
  B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&ctx->ev_free, cudaEventDisableTiming));
  return 0;
}

// Rows are independent, so the call is cut into row blocks and pipelined over three streams: while block i is
// computed, block i+1 is on its way in and block i-1 on its way out (PCIe is full duplex).  With page-locked host
// buffers the call then costs about one direction of the transfer instead of both plus the compute.
int b200q_linear_f32_host(b200q_ctx* ctx, const float* x_host, const int8_t* W_nk, const float* w_scales, const float* bias,
                          int act, int64_t M, int64_t N, int64_t K, float* out_host) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_linear_f32_host");
  if (int e = check_linear("b200q_linear_f32_host", x_host, W_nk, w_scales, act, M, N, K, out_host)) return e;
  B200Q_REQUIRE(K > 0 || M == 0, "b200q_linear_f32_host: rows of zero length have no range");
  if (M == 0 || N == 0) return 0;
  if (host_pipeline_ready(ctx)) return 1;
  if (ws_reserve(ctx, ctx->ws_stage_in, (size_t)M * K * sizeof(float))) return 1;
  if (ws_reserve(ctx, ctx->ws_stage_out, (size_t)M * N * sizeof(float))) return 1;
  if (ws_reserve(ctx, ctx->ws_q, (size_t)M * K)) return 1;
  if (ws_reserve(ctx, ctx->ws_scales, (size_t)M * sizeof(float))) return 1;
  float* x = (float*)ctx->ws_stage_in.ptr;
  float* y = (float*)ctx->ws_stage_out.ptr;
  int8_t* q = (int8_t*)ctx->ws_q.ptr;
  float* sc = (float*)ctx->ws_scales.ptr;
  // Row blocks of a multiple of 256 rows (one tile of the CTA-pair kernel), at most HOST_CHUNKS of them.
  int64_t rows = ((M + HOST_CHUNKS - 1) / HOST_CHUNKS + 255) / 256 * 256;
  if (rows < 1024) rows = 1024;
  // The workspaces may just have been (re)allocated on the compute stream: the copy streams start after that.
  B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_free, ctx->stream));
  B200Q_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream_h2d, ctx->ev_free, 0));
  B200Q_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream_d2h, ctx->ev_free, 0));
  // Ordinary (pageable) host arrays are staged through page-locked memory by the context's copy threads, row block by
  // row block and in step with the transfers; page-locked (or registered) arrays are handed to the copy engines as
  // they are.
  const bool stage_in = !host_pointer_is_page_locked(x_host), stage_out = !host_pointer_is_page_locked(out_host);
  const size_t in_block = (size_t)rows * K * sizeof(float), out_block = (size_t)rows * N * sizeof(float);
  if (stage_in || stage_out) {
    if (int e = host_staging_ready(ctx, stage_in ? in_block : 0, stage_out ? out_block : 0)) return e;
  }
  const int chunks = (int)((M + rows - 1) / rows);
  constexpr int LAG = HOST_SLOTS - 1;     // a block's result is copied out this many blocks after the block went in
  for (int c = 0; c < chunks + (stage_out ? LAG : 0); c++) {
    const int64_t m0 = (int64_t)c * rows;
    const int64_t mc = c < chunks ? ((M - m0 < rows) ? (M - m0) : rows) : 0;
    const int slot = c % HOST_SLOTS;
    // host copies of this turn: block c into the ring, block c - LAG out of it
    void* in_dst = nullptr;
    size_t in_n = 0;
    if (stage_in && c < chunks) {
      if (c >= HOST_SLOTS) B200Q_CHECK_CUDA(cudaEventSynchronize(ctx->ev_in[c - HOST_SLOTS]));   // the slot's last transfer has read it
      in_dst = (char*)ctx->pin_in + (size_t)slot * in_block;
      in_n = (size_t)mc * K * sizeof(float);
    }
    void* out_dst = nullptr;
    const void* out_src = nullptr;
    size_t out_n = 0;
    if (stage_out && c >= LAG) {
      const int d = c - LAG;
      const int64_t d0 = (int64_t)d * rows, dc = (M - d0 < rows) ? (M - d0) : rows;
      B200Q_CHECK_CUDA(cudaEventSynchronize(ctx->ev_out[d]));
      out_dst = out_host + d0 * N;
      out_src = (char*)ctx->pin_out + (size_t)(d % HOST_SLOTS) * out_block;
      out_n = (size_t)dc * N * sizeof(float);
    }
    if (in_n || out_n) host_stager_copy2(ctx->stager, in_dst, x_host + m0 * K, in_n, out_dst, out_src, out_n);
    if (c >= chunks) continue;
    const void* h2d_src = stage_in ? in_dst : (const void*)(x_host + m0 * K);
    B200Q_CHECK_CUDA(cudaMemcpyAsync(x + m0 * K, h2d_src, (size_t)mc * K * sizeof(float), cudaMemcpyHostToDevice, ctx->stream_h2d));
    B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_in[c], ctx->stream_h2d));
    B200Q_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_in[c], 0));
    if (int e = launch_quantize_per_token(ctx, x + m0 * K, mc, K, q + m0 * K, sc + m0, -127, 127)) return e;
    if (int e = linear_core(ctx, q + m0 * K, sc + m0, W_nk, w_scales, bias, act, mc, N, K, y + m0 * N, nullptr, 1.0)) return e;
    B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_done[c], ctx->stream));
    B200Q_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream_d2h, ctx->ev_done[c], 0));
    // (the slot of the ring this block's result lands in was copied out LAG blocks ago, before this point)
    void* d2h_dst = stage_out ? (void*)((char*)ctx->pin_out + (size_t)slot * out_block) : (void*)(out_host + m0 * N);
    B200Q_CHECK_CUDA(cudaMemcpyAsync(d2h_dst, y + m0 * N, (size_t)mc * N * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream_d2h));
    B200Q_CHECK_CUDA(cudaEventRecord(ctx->ev_out[c], ctx->stream_d2h));
  }
  B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream_d2h));
  B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  return 0;
}

// ---------------------------------------------------------------- captured steps
struct b200q_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  uint64_t kernels = 0;   // kernel launches recorded in it
};

int b200q_graph_begin(b200q_ctx* ctx) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(!ctx->capturing, "b200q_graph_begin: a recording is already in progress on this context");
  B200Q_REQUIRE(!ctx->profiling, "b200q_graph_begin: switch per-kernel profiling off first");
  B200Q_CHECK_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  ctx->capturing = true;
  ctx->capture_launches0 = ctx->launches;
  return 0;
}

int b200q_graph_end(b200q_ctx* ctx, b200q_graph** out) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(out != nullptr, "b200q_graph_end: null out pointer");
  *out = nullptr;
  B200Q_REQUIRE(ctx->capturing, "b200q_graph_end: no recording in progress");
  ctx->capturing = false;
  cudaGraph_t graph = nullptr;
  cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
  const uint64_t kernels = ctx->launches - ctx->capture_launches0;
  ctx->launches = ctx->capture_launches0;   // nothing ran: the recorded kernels count when the graph is launched
  if (e != cudaSuccess || !graph) {
    set_error("b200q_graph_end: the recording failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return 1;
  }
  cudaGraphExec_t exec = nullptr;
  e = cudaGraphInstantiate(&exec, graph, 0);
  if (e != cudaSuccess) {
    set_error("b200q_graph_end: cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    cudaGraphDestroy(graph);
    return 1;
  }
  b200q_graph* g = new (std::nothrow) b200q_graph();
  if (!g) {
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(graph);
    set_error("b200q_graph_end: out of host memory");
    return 2;
  }
  g->graph = graph;
  g->exec = exec;
  g->kernels = kernels;
  *out = g;
  return 0;
}

int b200q_graph_launch(b200q_ctx* ctx, b200q_graph* graph) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(graph != nullptr && graph->exec != nullptr, "b200q_graph_launch: null graph");
  B200Q_NOT_CAPTURING(ctx, "b200q_graph_launch");
  B200Q_CHECK_CUDA(cudaGraphLaunch(graph->exec, ctx->stream));
  ctx->launches += graph->kernels;
  return 0;
}

int b200q_graph_destroy(b200q_ctx* ctx, b200q_graph* graph) {
  if (use_device(ctx)) return 1;
  if (!graph) return 0;
  B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  if (graph->exec) cudaGraphExecDestroy(graph->exec);
  if (graph->graph) cudaGraphDestroy(graph->graph);
  delete graph;
  return 0;
}

int b200q_selftest_bounded_wait(b200q_ctx* ctx, double limit_seconds) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(limit_seconds > 0 && limit_seconds <= 1.0, "b200q_selftest_bounded_wait: %g s is outside (0, 1]", limit_seconds);
  return launch_selftest_bounded_wait(ctx, (unsigned long long)(limit_seconds * 1e9));
}

int b200q_observer_reset(b200q_ctx* ctx, float* state) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_observer_reset");
  B200Q_REQUIRE(state != nullptr, "b200q_observer_reset: null pointer");
  const float init[2] = {std::numeric_limits<float>::infinity(), -std::numeric_limits<float>::infinity()};
  B200Q_CHECK_CUDA(cudaMemcpyAsync(state, init, sizeof(init), cudaMemcpyHostToDevice, ctx->stream));
  B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));   // `init` lives on this stack frame
  return 0;
}

int b200q_observe_minmax(b200q_ctx* ctx, const float* x, int64_t n, float* state) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(n >= 0, "b200q_observe_minmax: negative length");
  B200Q_REQUIRE(state != nullptr && (n == 0 || x != nullptr), "b200q_observe_minmax: null pointer");
  return launch_minmax_observe(ctx, x, n, state);
}

int b200q_histogram_f32(b200q_ctx* ctx, const float* x, int64_t n, double range_min, double range_max, int num_bins,
                        uint64_t* bins) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(n >= 0, "b200q_histogram_f32: negative length");
  B200Q_REQUIRE(bins != nullptr && (n == 0 || x != nullptr), "b200q_histogram_f32: null pointer");
  return launch_histogram_f32(ctx, x, n, range_min, range_max, num_bins, reinterpret_cast<unsigned long long*>(bins));
}

// HistogramCollector.computePercentileThreshold (src/compiler/analysis/calibration.ts:130-141).
int b200q_histogram_percentile_threshold(const double* bins, int num_bins, double total_count, double range_min, double range_max,
                                         double percentile, double* threshold) {
  B200Q_REQUIRE(bins != nullptr && threshold != nullptr && num_bins >= 1, "b200q_histogram_percentile_threshold: bad argument");
  const double target = total_count * percentile;
  double cumulative = 0.0;
  const double bin_width = (range_max - range_min) / num_bins;
  for (int i = 0; i < num_bins; i++) {
    cumulative += bins[i];
    if (cumulative >= target) {
      *threshold = range_min + (i + 1) * bin_width;
      return 0;
    }
  }
  *threshold = range_max;
  return 0;
}

// HistogramCollector.computeEntropyThreshold (calibration.ts:143-186): the clipping point whose quantized
// distribution has the smallest KL divergence from the observed one; every sum in the reference's order.
int b200q_histogram_entropy_threshold(const double* bins, int num_bins, double total_count, double range_min, double range_max,
                                      int num_quant_bins, double* threshold) {
  B200Q_REQUIRE(bins != nullptr && threshold != nullptr && num_bins >= 1 && num_quant_bins >= 1,
                "b200q_histogram_entropy_threshold: bad argument");
  if (total_count == 0.0) {
    *threshold = range_max;
    return 0;
  }
  double* ref = new (std::nothrow) double[2 * (size_t)num_bins];
  B200Q_REQUIRE(ref != nullptr, "b200q_histogram_entropy_threshold: out of host memory");
  double* q = ref + num_bins;
  for (int i = 0; i < num_bins; i++) ref[i] = bins[i] / total_count;
  int best_idx = num_bins;
  double best_kl = std::numeric_limits<double>::infinity();
  for (int t = num_quant_bins; t <= num_bins; t++) {
    const double quant_bin_width = (double)t / (double)num_quant_bins;
    for (int i = 0; i < t; i++) q[i] = 0.0;
    for (int i = 0; i < num_quant_bins; i++) {
      const int start = (int)std::floor(i * quant_bin_width);
      int end = (int)std::floor((i + 1) * quant_bin_width);
      if (end > t) end = t;
      double sum = 0.0;
      for (int j = start; j < end; j++) sum += ref[j];
      const int bin_count = end - start;
      if (bin_count > 0) {
        const double avg = sum / bin_count;
        for (int j = start; j < end; j++) q[j] = avg;
      }
    }
    double kl = 0.0;
    for (int i = 0; i < t; i++)
      if (ref[i] > 0.0 && q[i] > 0.0) kl += ref[i] * std::log(ref[i] / q[i]);
    if (kl < best_kl) {
      best_kl = kl;
      best_idx = t;
    }
  }
  delete[] ref;
  const double bin_width = (range_max - range_min) / num_bins;
  *threshold = range_min + best_idx * bin_width;
  return 0;
}

int b200q_embedding_f32(b200q_ctx* ctx, const float* table, const int32_t* tokens, const float* pos_table, int64_t M, int64_t D,
                        int64_t V, int64_t S, float* out) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(M >= 0 && D >= 0 && V >= 0 && S >= 0, "b200q_embedding_f32: negative dimension");
  B200Q_REQUIRE(M == 0 || D == 0 || (table && tokens && out), "b200q_embedding_f32: null pointer");
  return launch_embedding(ctx, table, tokens, pos_table, M, D, V, S, out);
}

int b200q_add_f32(b200q_ctx* ctx, const float* a, const float* b, int64_t n, float* out) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(n >= 0, "b200q_add_f32: negative length");
  B200Q_REQUIRE(n == 0 || (a && b && out), "b200q_add_f32: null pointer");
  return launch_add_f32(ctx, a, b, n, out);
}

int b200q_layernorm_quantize(b200q_ctx* ctx, const float* x, const float* residual, const float* gamma, const float* beta,
                             float eps, int64_t M, int64_t D, float* sum_out, float* y_out, int8_t* q_out, float* scales_out) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(M >= 0 && D >= 0, "b200q_layernorm_quantize: negative dimension");
  B200Q_REQUIRE(M == 0 || (x && gamma && beta), "b200q_layernorm_quantize: null pointer");
  B200Q_REQUIRE(sum_out == nullptr || residual != nullptr, "b200q_layernorm_quantize: sum_out needs a residual");
  return launch_layernorm_quantize(ctx, x, residual, gamma, beta, eps, M, D, sum_out, y_out, q_out, scales_out);
}

int b200q_sdpa_f32(b200q_ctx* ctx, const float* q, const float* k, const float* v, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                   int64_t B, int64_t H, int64_t S, int64_t head_dim, float scale, int causal, float* out, int64_t ld_out) {
  if (use_device(ctx)) return 1;
  B200Q_REQUIRE(B >= 0 && H >= 0 && S >= 0, "b200q_sdpa_f32: negative dimension");
  B200Q_REQUIRE(B == 0 || H == 0 || S == 0 || (q && k && v && out), "b200q_sdpa_f32: null pointer");
  return launch_sdpa_f32(ctx, q, k, v, ld_q, ld_k, ld_v, B, H, S, head_dim, scale, causal, out, ld_out);
}

int b200q_quant_roundtrip_host(b200q_ctx* ctx, const float* x_host, int64_t M, int64_t K, int8_t* q_host, float* scales_host,
                               float* y_host) {
  if (use_device(ctx)) return 1;
  B200Q_NOT_CAPTURING(ctx, "b200q_quant_roundtrip_host");
  B200Q_DIMS_OK(M, 0, K);
  B200Q_REQUIRE(M == 0 || K == 0 || (x_host && y_host), "b200q_quant_roundtrip_host: null pointer");
  if (M == 0 || K == 0) return 0;
  const size_t n = (size_t)M * K;
  if (ws_reserve(ctx, ctx->ws_stage_in, n * sizeof(float))) return 1;
  if (ws_reserve(ctx, ctx->ws_stage_out, n * sizeof(float))) return 1;
  if (ws_reserve(ctx, ctx->ws_q, n)) return 1;
  if (ws_reserve(ctx, ctx->ws_scales, (size_t)M * sizeof(float))) return 1;
  float* x = (float*)ctx->ws_stage_in.ptr;
  float* y = (float*)ctx->ws_stage_out.ptr;
  int8_t* q = (int8_t*)ctx->ws_q.ptr;
  float* s = (float*)ctx->ws_scales.ptr;
  B200Q_CHECK_CUDA(cudaMemcpyAsync(x, x_host, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
  if (int e = launch_quantize_per_token(ctx, x, M, K, q, s, -127, 127)) return e;
  if (int e = launch_dequantize_per_token(ctx, q, s, M, K, y)) return e;
  if (q_host) B200Q_CHECK_CUDA(cudaMemcpyAsync(q_host, q, n, cudaMemcpyDeviceToHost, ctx->stream));
  if (scales_host) B200Q_CHECK_CUDA(cudaMemcpyAsync(scales_host, s, (size_t)M * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  B200Q_CHECK_CUDA(cudaMemcpyAsync(y_host, y, n * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
  B200Q_CHECK_CUDA(cudaStreamSynchronize(ctx->stream));
  return 0;
}

}  // extern "C"
