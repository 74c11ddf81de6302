// Several GPUs behind the C ABI: b200q_group_* (declared in include/b200q.h).
//
// The reference executes on one device (src/runtime/node/cuda/runtime_api.ts:16-18 hard-wires device 0; its
// all_gather / all_reduce graph ops decompose to single-device slices,
// src/compiler/passes/decompose/decomposition_pass.ts:105-143), so nothing here has a counterpart there.
//
// Two ways of sharding one quantized linear over the GPUs of a node:
//   * by rows (M): every GPU runs the ordinary b200q_linear_f32 on its own rows against replicated weights.  A row
//     depends on nothing but itself, so nothing is exchanged;
//   * by output channels (N): every GPU holds the int8 activations of ALL rows and the weights of its own channels.
//     Per layer: GEMM + tail on the local channels (the epilogue publishes every row's local range as keys), ONE
//     max-reduction of the 2*M keys over the GPUs (NCCL all-reduce), a one-pass encode of the local f32 columns with
//     the agreed range -- bit for bit the codes the whole row would get on one GPU -- and an NCCL all-gather of the
//     int8 column blocks (int8 on the wire, not f32).  The gathered buffer stays in the layout the all-gather leaves,
//     rank after rank; the next layer's GEMM reads it through a three-dimensional tensor map, so no re-layout pass
//     exists.  With more than one row chunk the collectives of chunk c run on a second stream while the GEMM of
//     chunk c+1 computes, and the next layer may start on chunk 0 while later chunks are still being gathered.
//
// NCCL is looked up at run time (dlopen of libnccl.so.2: the copy already in the process if there is one), so the
// library loads and every single-GPU entry point works where NCCL is absent.  One communicator per group.  A group is
// either made by one process for several of its GPUs (b200q_group_create: the process drives every rank, collectives
// are issued inside ncclGroupStart/End) or joined by one process per GPU (b200q_group_create_rank with a unique id
// that the ranks share by their own means).  Collectives are enqueued on CUDA streams; no call in here waits on the
// host except create, destroy and sync.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "../../include/b200q.h"
#include "common.cuh"
#include "kernels.cuh"

namespace {

using namespace b200q;

// The handful of NCCL declarations this file needs (public API of NCCL 2.x; values from its nccl.h).
typedef struct ncclComm* NcclComm;
struct NcclUniqueId { char internal[128]; };
enum { NCCL_INT8 = 0, NCCL_UINT8 = 1, NCCL_UINT32 = 3 };
enum { NCCL_MAX = 2 };

struct NcclApi {
  void* handle = nullptr;
  int (*GetVersion)(int*) = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*CommInitAll)(NcclComm*, int, const int*) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};

NcclApi g_nccl;

int nccl_api(NcclApi** out) {
  if (!g_nccl.handle) {
    // A copy that the process already holds comes first (two different NCCL builds in one process do not mix: a
    // host that will load its own later, as a Python process importing torch does, loads it before the first group
    // call or names it in B200Q_NCCL_LIBRARY); then the named one; then the system's.
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) {
      const char* named = getenv("B200Q_NCCL_LIBRARY");
      if (named && *named) {
        h = dlopen(named, RTLD_NOW | RTLD_GLOBAL);
        B200Q_REQUIRE(h != nullptr, "multi-GPU groups: B200Q_NCCL_LIBRARY=%s could not be loaded (%s)", named, dlerror());
      }
    }
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    B200Q_REQUIRE(h != nullptr, "multi-GPU groups need NCCL: libnccl.so.2 could not be loaded (%s)", dlerror());
    NcclApi a;
    a.handle = h;
#define B200Q_NCCL_SYM(field, name)                                                        \
  *reinterpret_cast<void**>(&a.field) = dlsym(h, name);                                     \
  B200Q_REQUIRE(a.field != nullptr, "multi-GPU groups need NCCL: %s is missing from libnccl", name)
    B200Q_NCCL_SYM(GetVersion, "ncclGetVersion");
    B200Q_NCCL_SYM(GetUniqueId, "ncclGetUniqueId");
    B200Q_NCCL_SYM(CommInitRank, "ncclCommInitRank");
    B200Q_NCCL_SYM(CommInitAll, "ncclCommInitAll");
    B200Q_NCCL_SYM(CommDestroy, "ncclCommDestroy");
    B200Q_NCCL_SYM(AllReduce, "ncclAllReduce");
    B200Q_NCCL_SYM(AllGather, "ncclAllGather");
    B200Q_NCCL_SYM(GroupStart, "ncclGroupStart");
    B200Q_NCCL_SYM(GroupEnd, "ncclGroupEnd");
    B200Q_NCCL_SYM(GetErrorString, "ncclGetErrorString");
#undef B200Q_NCCL_SYM
    g_nccl = a;
  }
  *out = &g_nccl;
  return 0;
}

#define B200Q_CHECK_NCCL(api, expr)                                                                      \
  do {                                                                                                   \
    int _r = (expr);                                                                                     \
    if (_r != 0) {                                                                                       \
      ::b200q::set_error("%s failed: %s (%s:%d)", #expr, (api)->GetErrorString(_r), __FILE__, __LINE__); \
      return 1;                                                                                          \
    }                                                                                                    \
  } while (0)

constexpr int MAX_CHUNKS = 16;

// What one rank driven by this process owns.
struct Member {
  b200q_ctx* ctx = nullptr;
  int rank = 0;
  NcclComm comm = nullptr;
  cudaStream_t comm_stream = nullptr;         // collectives of a chunked call; the context's stream otherwise
  Workspace y, keys;                          // f32 result of the local channels, range keys
  // Local codes, two buffers used in turn by successive calls: chunk c of one call sits at a different offset than
  // chunk c of the next (the channel counts differ), so a call must not write where the previous call's later
  // all-gathers may still be reading.  By the end of a call the context's stream has waited for every all-gather of
  // the call before it, which makes the buffer of two calls ago free again.
  Workspace q_local[2];
  int q_flip = 0;
  cudaEvent_t ev_gemm[MAX_CHUNKS] = {}, ev_reduced[MAX_CHUNKS] = {}, ev_coded[MAX_CHUNKS] = {}, ev_gathered[MAX_CHUNKS] = {};
  int gathers_pending = 0;                    // chunks of the previous channel-sharded call whose all-gather the context's stream has not waited for
};

}  // namespace

struct b200q_group {
  int world = 0;
  bool owns_contexts = false;
  int chunks = 1;
  NcclApi* api = nullptr;
  std::vector<Member> members;
};

namespace {

int member_reserve(Member& m, Workspace& ws, size_t bytes) { return ws_reserve(m.ctx, ws, bytes); }

int member_events(Member& m) {
  if (m.ev_gemm[0]) return 0;
  B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
  B200Q_CHECK_CUDA(cudaStreamCreateWithFlags(&m.comm_stream, cudaStreamNonBlocking));
  for (int c = 0; c < MAX_CHUNKS; c++) {
    B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&m.ev_gemm[c], cudaEventDisableTiming));
    B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&m.ev_reduced[c], cudaEventDisableTiming));
    B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&m.ev_coded[c], cudaEventDisableTiming));
    B200Q_CHECK_CUDA(cudaEventCreateWithFlags(&m.ev_gathered[c], cudaEventDisableTiming));
  }
  return 0;
}

// Rows of chunk c of M rows cut into `chunks` pieces of whole 256-row tiles (the last one takes what is left).
void chunk_rows(int64_t M, int chunks, int c, int64_t* r0, int64_t* rows) {
  int64_t per = ((M + chunks - 1) / chunks + 255) / 256 * 256;
  int64_t a = per * c, b = a + per;
  if (a > M) a = M;
  if (b > M) b = M;
  *r0 = a;
  *rows = b - a;
}

// The context's stream waits for every all-gather of the previous chunked call that it has not yet waited for.
int fence_member(Member& m) {
  for (int c = 0; c < m.gathers_pending; c++) B200Q_CHECK_CUDA(cudaStreamWaitEvent(m.ctx->stream, m.ev_gathered[c], 0));
  m.gathers_pending = 0;
  return 0;
}

}  // namespace

extern "C" {

int b200q_group_unique_id(void* id128) {
  B200Q_REQUIRE(id128 != nullptr, "b200q_group_unique_id: null pointer");
  NcclApi* api = nullptr;
  if (int e = nccl_api(&api)) return e;
  NcclUniqueId id;
  B200Q_CHECK_NCCL(api, api->GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return 0;
}

int b200q_group_create(const int* devices, int n, b200q_group** out) {
  B200Q_REQUIRE(out != nullptr, "b200q_group_create: null out pointer");
  *out = nullptr;
  B200Q_REQUIRE(devices != nullptr && n >= 1 && n <= 64, "b200q_group_create: need 1 to 64 device ordinals");
  for (int i = 0; i < n; i++)
    for (int j = 0; j < i; j++) B200Q_REQUIRE(devices[i] != devices[j], "b200q_group_create: device %d is listed twice", devices[i]);
  NcclApi* api = nullptr;
  if (int e = nccl_api(&api)) return e;
  b200q_group* g = new (std::nothrow) b200q_group();
  B200Q_REQUIRE(g != nullptr, "b200q_group_create: out of host memory");
  g->world = n;
  g->owns_contexts = true;
  g->api = api;
  g->members.resize(n);
  for (int i = 0; i < n; i++) {
    g->members[i].rank = i;
    if (int e = b200q_create(devices[i], &g->members[i].ctx)) {
      b200q_group_destroy(g);
      return e;
    }
  }
  std::vector<NcclComm> comms(n, nullptr);
  int r = api->CommInitAll(comms.data(), n, devices);
  if (r != 0) {
    set_error("ncclCommInitAll failed: %s", api->GetErrorString(r));
    b200q_group_destroy(g);
    return 1;
  }
  for (int i = 0; i < n; i++) g->members[i].comm = comms[i];
  *out = g;
  return 0;
}

int b200q_group_create_rank(b200q_ctx* ctx, const void* id128, int rank, int world, b200q_group** out) {
  B200Q_REQUIRE(out != nullptr, "b200q_group_create_rank: null out pointer");
  *out = nullptr;
  B200Q_REQUIRE(ctx != nullptr && id128 != nullptr, "b200q_group_create_rank: null context or id");
  B200Q_REQUIRE(world >= 1 && rank >= 0 && rank < world, "b200q_group_create_rank: rank %d of %d", rank, world);
  NcclApi* api = nullptr;
  if (int e = nccl_api(&api)) return e;
  B200Q_CHECK_CUDA(cudaSetDevice(ctx->device));
  NcclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  NcclComm comm = nullptr;
  B200Q_CHECK_NCCL(api, api->CommInitRank(&comm, world, id, rank));
  b200q_group* g = new (std::nothrow) b200q_group();
  if (!g) {
    api->CommDestroy(comm);
    set_error("b200q_group_create_rank: out of host memory");
    return 2;
  }
  g->world = world;
  g->owns_contexts = false;
  g->api = api;
  g->members.resize(1);
  g->members[0].ctx = ctx;
  g->members[0].rank = rank;
  g->members[0].comm = comm;
  *out = g;
  return 0;
}

int b200q_group_destroy(b200q_group* g) {
  if (!g) return 0;
  for (Member& m : g->members) {
    if (!m.ctx) continue;
    cudaSetDevice(m.ctx->device);
    if (m.comm_stream) cudaStreamSynchronize(m.comm_stream);
    cudaStreamSynchronize(m.ctx->stream);
  }
  for (Member& m : g->members)
    if (m.comm) g->api->CommDestroy(m.comm);
  for (Member& m : g->members) {
    if (!m.ctx) continue;
    cudaSetDevice(m.ctx->device);
    Workspace* all[] = {&m.y, &m.keys, &m.q_local[0], &m.q_local[1]};
    for (Workspace* w : all)
      if (w->ptr) cudaFree(w->ptr);
    for (int c = 0; c < MAX_CHUNKS; c++) {
      if (m.ev_gemm[c]) cudaEventDestroy(m.ev_gemm[c]);
      if (m.ev_reduced[c]) cudaEventDestroy(m.ev_reduced[c]);
      if (m.ev_coded[c]) cudaEventDestroy(m.ev_coded[c]);
      if (m.ev_gathered[c]) cudaEventDestroy(m.ev_gathered[c]);
    }
    if (m.comm_stream) cudaStreamDestroy(m.comm_stream);
    if (g->owns_contexts) b200q_destroy(m.ctx);
  }
  delete g;
  return 0;
}

int b200q_group_world(b200q_group* g) { return g ? g->world : 0; }
int b200q_group_local_count(b200q_group* g) { return g ? (int)g->members.size() : 0; }
b200q_ctx* b200q_group_ctx(b200q_group* g, int i) { return (g && i >= 0 && i < (int)g->members.size()) ? g->members[i].ctx : nullptr; }
int b200q_group_rank(b200q_group* g, int i) { return (g && i >= 0 && i < (int)g->members.size()) ? g->members[i].rank : -1; }

int b200q_group_nccl_version(b200q_group* g, int* version) {
  B200Q_REQUIRE(g != nullptr && version != nullptr, "b200q_group_nccl_version: null pointer");
  B200Q_CHECK_NCCL(g->api, g->api->GetVersion(version));
  return 0;
}

int b200q_group_set_chunks(b200q_group* g, int chunks) {
  B200Q_REQUIRE(g != nullptr, "null group");
  B200Q_REQUIRE(chunks >= 1 && chunks <= MAX_CHUNKS, "b200q_group_set_chunks: %d is outside [1, %d]", chunks, MAX_CHUNKS);
  for (Member& m : g->members)
    if (int e = fence_member(m)) return e;
  g->chunks = chunks;
  return 0;
}

int b200q_group_fence(b200q_group* g) {
  B200Q_REQUIRE(g != nullptr, "null group");
  for (Member& m : g->members) {
    B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
    if (int e = fence_member(m)) return e;
  }
  return 0;
}

int b200q_group_sync(b200q_group* g) {
  B200Q_REQUIRE(g != nullptr, "null group");
  for (Member& m : g->members) {
    B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
    if (int e = fence_member(m)) return e;
    B200Q_CHECK_CUDA(cudaStreamSynchronize(m.ctx->stream));
  }
  return 0;
}

int b200q_group_linear_mshard(b200q_group* g, const float* const* x, const int64_t* rows, const int8_t* const* W_nk,
                              const float* const* w_scales, const float* const* bias, int act, int64_t N, int64_t K,
                              float* const* out) {
  B200Q_REQUIRE(g != nullptr, "null group");
  B200Q_REQUIRE(x && rows && W_nk && w_scales && out, "b200q_group_linear_mshard: null argument array");
  for (size_t i = 0; i < g->members.size(); i++) {
    if (int e = b200q_linear_f32(g->members[i].ctx, x[i], W_nk[i], w_scales[i], bias ? bias[i] : nullptr, act, rows[i], N, K, out[i]))
      return e;
  }
  return 0;
}

int b200q_group_all_gather(b200q_group* g, const void* const* send, void* const* recv, size_t bytes) {
  B200Q_REQUIRE(g != nullptr, "null group");
  B200Q_REQUIRE(send && recv, "b200q_group_all_gather: null argument array");
  if (bytes == 0) return 0;
  NcclApi* api = g->api;
  const bool many = g->members.size() > 1;
  if (many) B200Q_CHECK_NCCL(api, api->GroupStart());
  for (size_t i = 0; i < g->members.size(); i++) {
    Member& m = g->members[i];
    B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
    if (int e = fence_member(m)) return e;
    B200Q_CHECK_NCCL(api, api->AllGather(send[i], recv[i], bytes, NCCL_INT8, m.comm, m.ctx->stream));
  }
  if (many) B200Q_CHECK_NCCL(api, api->GroupEnd());
  return 0;
}

int b200q_group_linear_nshard(b200q_group* g, const int8_t* const* q_in, const float* const* in_scales, int in_blocks,
                              const int8_t* const* W_shard, const float* const* w_scales, const float* const* bias, int act,
                              int64_t M, int64_t N, int64_t K, int8_t* const* q_out, float* const* out_scales,
                              float* const* out_f32) {
  B200Q_REQUIRE(g != nullptr, "null group");
  B200Q_REQUIRE(q_in && in_scales && W_shard && w_scales, "b200q_group_linear_nshard: null argument array");
  B200Q_REQUIRE((q_out != nullptr && out_scales != nullptr) != (out_f32 != nullptr),
                "b200q_group_linear_nshard: give either q_out and out_scales (requantized, gathered) or out_f32 (local channels)");
  B200Q_REQUIRE(M >= 0 && N >= 0 && K > 0, "b200q_group_linear_nshard: bad dimension (M=%lld N=%lld K=%lld)", (long long)M,
                (long long)N, (long long)K);
  B200Q_REQUIRE(act >= 0 && act <= 4, "b200q_group_linear_nshard: unknown activation %d", act);
  const int W = g->world;
  B200Q_REQUIRE(N % W == 0, "b200q_group_linear_nshard: N=%lld does not split evenly over %d GPUs", (long long)N, W);
  const int64_t cols = N / W;
  B200Q_REQUIRE(in_blocks == 1 || in_blocks == W, "b200q_group_linear_nshard: the input is row-major (1) or gathered from %d GPUs, not %d blocks",
                W, in_blocks);
  B200Q_REQUIRE(q_out == nullptr || W == 1 || cols % 128 == 0,
                "b200q_group_linear_nshard: gathered int8 output needs a multiple of 128 channels per GPU (N=%lld over %d GPUs gives %lld)",
                (long long)N, W, (long long)cols);
  if (M == 0 || N == 0) return 0;
  NcclApi* api = g->api;
  const size_t nm = g->members.size();
  const bool many = nm > 1;
  const int chunks = g->chunks;
  const bool side = chunks > 1 && W > 1 && q_out != nullptr;   // collectives on their own stream
  for (size_t i = 0; i < nm; i++) {
    Member& m = g->members[i];
    B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
    if (side) {
      if (int e = member_events(m)) return e;
    }
    if (q_out) {
      // A workspace that has to grow is freed in the order of the context's stream, which knows nothing of the
      // collectives still running on the second stream: wait for those first (sizes settle after the first pass).
      const bool grows = (size_t)M * cols * sizeof(float) > m.y.bytes || (size_t)2 * M * sizeof(uint32_t) > m.keys.bytes ||
                         (W > 1 && ((size_t)M * cols > m.q_local[0].bytes || (size_t)M * cols > m.q_local[1].bytes));
      if (grows) {
        if (int e = fence_member(m)) return e;
      }
      if (member_reserve(m, m.y, (size_t)M * cols * sizeof(float))) return 1;
      if (member_reserve(m, m.keys, (size_t)2 * M * sizeof(uint32_t))) return 1;
      if (W > 1 && (member_reserve(m, m.q_local[0], (size_t)M * cols) || member_reserve(m, m.q_local[1], (size_t)M * cols))) return 1;
      m.q_flip ^= 1;
      B200Q_CHECK_CUDA(cudaMemsetAsync(m.keys.ptr, 0, (size_t)2 * M * sizeof(uint32_t), m.ctx->stream));
    }
  }
  // Row chunk by row chunk; every phase is issued for all local ranks before the next begins, so that the
  // collectives of the ranks of one process sit together inside ncclGroupStart / ncclGroupEnd.
  for (int c = 0; c < chunks; c++) {
    int64_t r0, rc;
    chunk_rows(M, chunks, c, &r0, &rc);
    if (rc == 0) continue;
    // Where the chunk's rows start in a buffer gathered from `W` GPUs: chunks follow each other, and inside a chunk
    // the column blocks of the ranks follow each other ([chunk][rank][rows of the chunk][cols]).
    for (size_t i = 0; i < nm; i++) {
      Member& m = g->members[i];
      b200q_ctx* ctx = m.ctx;
      B200Q_CHECK_CUDA(cudaSetDevice(ctx->device));
      // this chunk of the input was gathered by the previous call's collectives
      if (c < m.gathers_pending) B200Q_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream, m.ev_gathered[c], 0));
      const int8_t* a = q_in[i] + r0 * K;   // row-major: rows r0..; gathered: in_blocks * (K / in_blocks) * r0 = K * r0 as well
      const float* a_sc = in_scales[i] + r0;
      const float* b = bias ? bias[i] : nullptr;
      if (out_f32) {
        if (!gemm_umma_supported(a, W_shard[i], rc, cols, K) || ctx->gemm_variant == 1) {
          B200Q_REQUIRE(in_blocks == 1, "b200q_group_linear_nshard: a gathered input needs the tensor-core kernel (K %% 16 == 0, aligned operands)");
          if (int e = b200q_int8_linear(ctx, a, a_sc, W_shard[i], w_scales[i], b, act, rc, cols, K, out_f32[i] + r0 * cols)) return e;
        } else if (int e = launch_gemm_i8_umma(ctx, a, W_shard[i], rc, cols, K, a_sc, w_scales[i], b, act, out_f32[i] + r0 * cols, nullptr,
                                               nullptr, 1.0, nullptr, in_blocks)) {
          return e;
        }
        continue;
      }
      float* y = (float*)m.y.ptr + r0 * cols;
      uint32_t* keys = (uint32_t*)m.keys.ptr + 2 * r0;
      B200Q_REQUIRE(gemm_umma_supported(a, W_shard[i], rc, cols, K) && ctx->gemm_variant != 1,
                    "b200q_group_linear_nshard: the requantized form needs the tensor-core kernel (K %% 16 == 0, aligned operands)");
      if (int e = launch_gemm_i8_umma(ctx, a, W_shard[i], rc, cols, K, a_sc, w_scales[i], b, act, y, nullptr, nullptr, 1.0, keys, in_blocks))
        return e;
      if (side) B200Q_CHECK_CUDA(cudaEventRecord(m.ev_gemm[c], ctx->stream));
    }
    if (out_f32) continue;
    // the rows' ranges over all GPUs: one max-reduction of the keys
    if (W > 1) {
      if (many) B200Q_CHECK_NCCL(api, api->GroupStart());
      for (size_t i = 0; i < nm; i++) {
        Member& m = g->members[i];
        B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
        cudaStream_t cs = side ? m.comm_stream : m.ctx->stream;
        if (side) B200Q_CHECK_CUDA(cudaStreamWaitEvent(cs, m.ev_gemm[c], 0));
        uint32_t* keys = (uint32_t*)m.keys.ptr + 2 * r0;
        B200Q_CHECK_NCCL(api, api->AllReduce(keys, keys, (size_t)2 * rc, NCCL_UINT32, NCCL_MAX, m.comm, cs));
      }
      if (many) B200Q_CHECK_NCCL(api, api->GroupEnd());
      // Inside a group the collectives reach their streams only at ncclGroupEnd: an event recorded before that would
      // not cover them.
      if (side) {
        for (size_t i = 0; i < nm; i++) {
          Member& m = g->members[i];
          B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
          B200Q_CHECK_CUDA(cudaEventRecord(m.ev_reduced[c], m.comm_stream));
        }
      }
    }
    // codes of the local channels from the agreed range
    for (size_t i = 0; i < nm; i++) {
      Member& m = g->members[i];
      b200q_ctx* ctx = m.ctx;
      B200Q_CHECK_CUDA(cudaSetDevice(ctx->device));
      if (side) B200Q_CHECK_CUDA(cudaStreamWaitEvent(ctx->stream, m.ev_reduced[c], 0));
      const float* y = (const float*)m.y.ptr + r0 * cols;
      const uint32_t* keys = (const uint32_t*)m.keys.ptr + 2 * r0;
      int8_t* dst = W > 1 ? (int8_t*)m.q_local[m.q_flip].ptr + r0 * cols : q_out[i] + r0 * N;
      if (int e = launch_quantize_rows_with_keys(ctx, y, rc, cols, cols, keys, dst, cols, out_scales[i] + r0, -127, 127)) return e;
      if (side) B200Q_CHECK_CUDA(cudaEventRecord(m.ev_coded[c], ctx->stream));
    }
    // int8 column blocks of every GPU, rank after rank
    if (W > 1) {
      if (many) B200Q_CHECK_NCCL(api, api->GroupStart());
      for (size_t i = 0; i < nm; i++) {
        Member& m = g->members[i];
        B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
        cudaStream_t cs = side ? m.comm_stream : m.ctx->stream;
        if (side) B200Q_CHECK_CUDA(cudaStreamWaitEvent(cs, m.ev_coded[c], 0));
        const int8_t* src = (const int8_t*)m.q_local[m.q_flip].ptr + r0 * cols;
        B200Q_CHECK_NCCL(api, api->AllGather(src, q_out[i] + r0 * N, (size_t)rc * cols, NCCL_INT8, m.comm, cs));
      }
      if (many) B200Q_CHECK_NCCL(api, api->GroupEnd());
      if (side) {
        for (size_t i = 0; i < nm; i++) {
          Member& m = g->members[i];
          B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
          B200Q_CHECK_CUDA(cudaEventRecord(m.ev_gathered[c], m.comm_stream));
        }
      }
    }
  }
  for (size_t i = 0; i < nm; i++) {
    Member& m = g->members[i];
    if (out_f32) {
      // every chunk's wait was issued above only up to `chunks`; a previous call with more chunks leaves the rest here
      B200Q_CHECK_CUDA(cudaSetDevice(m.ctx->device));
      if (int e = fence_member(m)) return e;
    } else {
      m.gathers_pending = side ? chunks : 0;
    }
  }
  return 0;
}

}  // extern "C"
