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
// For them the scratch lives in the fixed array below, which is part of the library image.
// It is static device memory of this translation unit's CUDA module: a copy exists on each
// device on which this process has a CUDA context that has loaded the module, and it goes
// away when that context is destroyed (normally at process exit).  b200q_create looks the
// array's address up for the context's device (noalloc_prepare below), so the module is
// loaded - and its 4 MiB + 64 KiB reserved - when the context is created, never inside a
// call of this entry point.  A process that only creates contexts on GPU 0 holds nothing on
// the other GPUs.  The array is there whether or not this entry point is ever called, which
// is why it is small.
//
// Limits (rejected with an error otherwise): M * K <= B200Q_NOALLOC_MAX_CODES (4 Mi activation
// elements, e.g. 1024 x 4096) and M <= B200Q_NOALLOC_MAX_ROWS (16384); the shape must be one the
// tensor-core kernel takes (K a multiple of 16, 16-byte aligned operands), because the CUDA-core
// fallback needs a second, larger workspace.
//
// The array is shared by every call on a GPU and keeps whatever the last call left in it.
// Nothing in it has to start at zero: the quantize kernel writes every code and every scale
// that the GEMM of the same call reads.  Calls on ONE context follow each other on its stream
// and may be enqueued back to back without a synchronisation in between (the GEMM of call n
// completes before the quantize kernel of call n+1 touches the array: the dependent-launch
// wait of the quantize kernels comes before their first access).  Two calls that overlap on
// the same GPU (two contexts, i.e. two streams) race on it: issue them one after the other.
//
// In host code the array's name is only a stand-in of the host compiler, not a device
// address, so it is never passed to a kernel directly: noalloc_prepare asks the runtime for
// the array's address on a device (with that device current) and caches it per device ordinal.
//
// What "allocates nothing" covers: no cudaMalloc / cudaFree / stream-ordered allocation and no
// allocating library routine is called here or in the launchers below it.  The CUDA runtime
// itself loads a kernel's code the first time that kernel is launched, and each kernel
// instance (one per activation, per tile form: M below or from 1024 rows, per row-length class
// of the quantize kernel) has its shared-memory attribute set on first use.  A host that needs
// even those first-use steps out of the way (a pool that owns all of the device's memory, a
// stream capture) makes one warm-up call per activation and shape class it will use, before
// handing the device to its pool or beginning a capture.
#include <atomic>

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

// Device address of the array, per CUDA device ordinal (null = not looked up yet).  Contexts on
// different host threads may run the lookup at the same time; they store the same value.
static std::atomic<NoAllocScratch*> g_scratch_addr[B200Q_NOALLOC_MAX_DEVICES];

int scratch_for_device(int device, NoAllocScratch** out) {
  B200Q_REQUIRE(device >= 0 && device < B200Q_NOALLOC_MAX_DEVICES, "b200q_linear_f32_noalloc: device ordinal %d is not supported",
                device);
  NoAllocScratch* addr = g_scratch_addr[device].load(std::memory_order_relaxed);
  if (!addr) {
    void* p = nullptr;
    B200Q_CHECK_CUDA(cudaSetDevice(device));
    B200Q_CHECK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    B200Q_REQUIRE(p != nullptr, "b200q_linear_f32_noalloc: the scratch array has no address on device %d", device);
    addr = static_cast<NoAllocScratch*>(p);
    g_scratch_addr[device].store(addr, std::memory_order_relaxed);
  }
  *out = addr;
  return 0;
}

}  // namespace

// Called by b200q_create with the context's device current: loads this module on the device (which is what
// reserves the array there) and caches the array's address, so that the entry point below finds it ready.
// Ordinals beyond the cache are left alone (the entry point then reports them).
int b200q::noalloc_prepare(int device) {
  if (device < 0 || device >= B200Q_NOALLOC_MAX_DEVICES) return 0;
  NoAllocScratch* unused = nullptr;
  return scratch_for_device(device, &unused);
}

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
  // written without the product M * K, which can overflow for absurd K
  B200Q_REQUIRE(M <= B200Q_NOALLOC_MAX_ROWS && K <= B200Q_NOALLOC_MAX_CODES && M <= B200Q_NOALLOC_MAX_CODES / K,
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
