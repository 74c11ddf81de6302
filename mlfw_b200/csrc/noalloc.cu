// b200q_linear_f32_noalloc: the quantized linear for callers that must not allocate.
//
// b200q_linear_f32 keeps the int8 codes and per-token scales of its activations in a
// workspace that the context grows on demand with the CUDA allocator.  Some users of
// this library cannot have that happen inside the call:
//   * a host whose memory manager has taken the whole device up front and hands out
//     sub-ranges itself (the reference's own CUDA runtime pools device memory this way,
//     src/runtime/node/cuda/memory.ts) - a second allocator asking the driver for memory
//     fails or fragments what the pool believes it owns;
//   * a latency-bound serving loop, where an allocation may synchronise the device and
//     stall every stream for milliseconds;
//   * code running in a phase in which the CUDA allocation calls are not permitted at all.
// For them the scratch lives in the fixed array below, which is part of the library image:
// every GPU that loads libb200q.so holds it from load until the process exits, whether or
// not this entry point is ever called.  That is why it is small.
//
// Limits (rejected with an error otherwise): M * K <= B200Q_NOALLOC_MAX_CODES (4 Mi activation
// elements, e.g. 1024 x 4096) and M <= B200Q_NOALLOC_MAX_ROWS (16384); the shape must be one the
// tensor-core kernel takes (K a multiple of 16, 16-byte aligned operands), because the CUDA-core
// fallback needs a second, larger workspace.
//
// The array is shared by every call on a GPU and keeps whatever the last call left in it.
// Nothing in it has to start at zero: the quantize kernel writes every code and every scale
// that the GEMM of the same call reads.  Two calls that overlap on the same GPU (two contexts,
// i.e. two streams) race on it: issue them one after the other.
//
// In host code the array's name is only a stand-in of the host compiler, not a device
// address, so it is never passed to a kernel directly: the first call on each device asks the
// runtime for the array's address on that device (with that device current) and caches it.
// That first call does this one-time set-up; make it before any stream capture is begun.
#include "../../include/b200q.h"
#include "common.cuh"
#include "kernels.cuh"

#define B200Q_NOALLOC_MAX_CODES (4ll * 1024 * 1024)
#define B200Q_NOALLOC_MAX_ROWS 16384ll
#define B200Q_NOALLOC_MAX_DEVICES 64

namespace {

struct NoAllocScratch {
  int8_t codes[B200Q_NOALLOC_MAX_CODES];   // int8 activations [M,K]
  float scales[B200Q_NOALLOC_MAX_ROWS];    // per-token scales [M]
};

static __device__ __align__(256) NoAllocScratch g_noalloc_scratch;

// Device address of the array, per CUDA device ordinal (0 = not looked up yet).
static NoAllocScratch* g_scratch_addr[B200Q_NOALLOC_MAX_DEVICES] = {};

int scratch_for_device(int device, NoAllocScratch** out) {
  B200Q_REQUIRE(device >= 0 && device < B200Q_NOALLOC_MAX_DEVICES, "b200q_linear_f32_noalloc: device ordinal %d is not supported",
                device);
  if (!g_scratch_addr[device]) {
    void* p = nullptr;
    B200Q_CHECK_CUDA(cudaSetDevice(device));
    B200Q_CHECK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    B200Q_REQUIRE(p != nullptr, "b200q_linear_f32_noalloc: the scratch array has no address on device %d", device);
    g_scratch_addr[device] = static_cast<NoAllocScratch*>(p);
  }
  *out = g_scratch_addr[device];
  return 0;
}

}  // namespace

extern "C" int b200q_linear_f32_noalloc(b200q_ctx* ctx, const float* x, const int8_t* W_nk, const float* w_scales,
                                        const float* bias, int act, int64_t M, int64_t N, int64_t K, float* out) {
  using namespace b200q;
  B200Q_REQUIRE(ctx != nullptr, "null context");
  B200Q_CHECK_CUDA(cudaSetDevice(ctx->device));
  B200Q_REQUIRE(M >= 0 && N >= 0 && K >= 0, "b200q_linear_f32_noalloc: negative dimension (M=%lld N=%lld K=%lld)", (long long)M,
                (long long)N, (long long)K);
  B200Q_REQUIRE(act >= 0 && act <= 4, "b200q_linear_f32_noalloc: unknown activation %d", act);
  if (M == 0 || N == 0) return 0;
  B200Q_REQUIRE(x && W_nk && w_scales && out, "b200q_linear_f32_noalloc: null pointer");
  B200Q_REQUIRE(K > 0, "b200q_linear_f32_noalloc: rows of zero length have no range");
  B200Q_REQUIRE(M <= B200Q_NOALLOC_MAX_ROWS && M * K <= B200Q_NOALLOC_MAX_CODES,
                "b200q_linear_f32_noalloc: M=%lld K=%lld exceeds the fixed scratch (at most %lld rows and %lld activation elements); "
                "use b200q_linear_f32",
                (long long)M, (long long)K, (long long)B200Q_NOALLOC_MAX_ROWS, (long long)B200Q_NOALLOC_MAX_CODES);
  NoAllocScratch* scratch = nullptr;
  if (int e = scratch_for_device(ctx->device, &scratch)) return e;
  B200Q_REQUIRE(ctx->gemm_variant != 1 && gemm_umma_supported(scratch->codes, W_nk, M, N, K),
                "b200q_linear_f32_noalloc: this shape needs the CUDA-core kernel and its workspace (K must be a multiple of 16 "
                "and the weights 16-byte aligned); use b200q_linear_f32");
  if (int e = launch_quantize_per_token(ctx, x, M, K, scratch->codes, scratch->scales, -127, 127)) return e;
  return launch_gemm_i8_umma(ctx, scratch->codes, W_nk, M, N, K, scratch->scales, w_scales, bias, act, out, nullptr, nullptr, 1.0);
}
