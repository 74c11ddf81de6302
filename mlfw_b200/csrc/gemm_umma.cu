// int8 x int8 -> int32 GEMM on the 5th-generation tensor cores with the whole
// quantized-linear tail fused into the epilogue.
//
//   C[m,n] = sum_k A[m,k] * W[n,k]                    (tcgen05.mma.kind::i8, int32 in tensor memory)
//   y      = act( C * (aScale[m] * wScale[n]) + bias[n] )     -> f32, or
//   q      = static requantization of y                        -> int8, or
//   C                                                           -> int32
//
// Reference semantics: quantized_dot (src/compiler/passes/lowering/rules/
// quantization.ts:23-42) followed by the per-channel tail the quantization pass
// emits (src/compiler/passes/quantization/quantization_pass.ts:427-456), bias
// (src/nn/functional/linear.ts:13-15) and the decomposed activation.  Fusing is a
// performance change only: the arithmetic is the same chain, rounded at the
// same points (see quant_math.cuh).
//
// Two variants share the code: one CTA per 128x256 tile (cta_group::1), and a pair of CTAs on
// neighbouring SMs per 256x256 tile (cta_group::2: each CTA stages its own 128 rows of A and its own
// half of the W tile, one thread of the even CTA issues MMAs that span both SMs; this cuts the L2 ->
// shared-memory traffic per output by a third and halves the W reads of each SM's tensor core).
// No load is multicast: every CTA fetches its own operands.
//
// Structure (one CTA per SM, persistent over its tiles):
//   warp 0     TMA producer: A tile 128x128 B and W tile 256x128 B per stage, 128-byte swizzle
//   warp 1     allocates tensor memory, one lane issues tcgen05.mma (4 per stage, K = 32 each)
//   warps 2-9  epilogue: tcgen05.ld of a finished accumulator, tail arithmetic, global stores
//              (warp w reads tensor-memory lanes 32*(w%4).., i.e. 32 rows, and half of the columns)
// The accumulator is double buffered in tensor memory (2 x 256 columns), so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Every wait is bounded: a role that waits longer than the context's limit sets a
// bit in the status word, raises a CTA-wide abort flag and all roles leave their
// loops; the CTA then lets copies in flight land, frees tensor memory and returns.
#include <cuda.h>

#include <cstddef>

#include "common.cuh"
#include "kernels.cuh"
#include "quant_math.cuh"

namespace b200q {

namespace {

constexpr int BM = 128, BN = 256, BK = 128;  // per-CTA tile; int8: bytes == elements
constexpr int UMMA_K = 32;
constexpr int MAX_STAGES = 6;
// EW epilogue warps: 8 (two per tensor-memory lane quarter, 128 columns of a tile each) or 16 (four per quarter, 64
// columns each).  Sixteen hide the latencies of the epilogue's chain (tensor-memory load, staging, proxy fence, bulk
// store) twice as well and are used where the epilogue, not the tensor pipe, sets the pace: short K.  They cost one
// operand stage (their staging tiles) and leave 113 registers per thread.
template <int NCTA, int EW = 8>
struct Cfg {
  static constexpr int B_ROWS = BN / NCTA;  // rows of the W tile one CTA stages
  static constexpr int A_BYTES = BM * BK, B_BYTES = B_ROWS * BK, STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (NCTA == 1 ? 4 : 6) - (EW == 16 ? 1 : 0);
  static constexpr int EPI_COLS = BN / (EW / 4);   // columns of a tile one epilogue warp handles
  static constexpr int THREADS = 64 + 32 * EW;
};
constexpr int MAX_EPI_WARPS = 16;
constexpr int TMEM_COLS = 512;
constexpr int EPI_CH = 16;                     // columns an epilogue warp takes from tensor memory at a time
// Staging tile of one epilogue warp for the bulk-tensor store of a chunk: 32 rows x EPI_CH 4-byte values.
constexpr int OUT_STAGE_BYTES = 32 * EPI_CH * 4;
constexpr int MISC_BYTES = 3584 + 4 * BN * 8;     // per-warp column scales and biases: EW * EPI_COLS = 4 * BN floats each
template <int NCTA, int EW = 8>
constexpr int smem_bytes() {  // + slack to align the tiles to 1024 B
  return Cfg<NCTA, EW>::STAGES * Cfg<NCTA, EW>::STAGE_BYTES + EW * OUT_STAGE_BYTES + MISC_BYTES + 1024;
}

struct GemmParams {
  int64_t M, N, K;
  const float* a_scales;  // [M] or null
  const float* w_scales;  // [N]; null when the raw accumulator is the output
  const float* bias;      // [N] or null
  int act;
  float* out_f32;
  int32_t* out_i32;
  int8_t* out_q;
  double q_scale;
  float q_inv;
  int q_exact;
  // What the contraction length guarantees about the accumulators (|a|, |w| <= 128): 0: below 2^22 (K <= 255), the
  // conversion without a conversion instruction is exact; 1: at most 2^24 (K <= 1024), the conversion instruction is
  // exact; 2: nothing, every chunk tests its accumulators and goes through binary64 when one reaches 2^22.
  int acc_class;
  int tma_store;          // results leave through bulk-tensor stores (needs a 16-byte aligned base and row pitch)
  // f32 output only: when not null, the NaN-ignoring maximum and minimum of every output row are published here as
  // order-preserving keys (range_key_max / range_key_min in quant_math.cuh), [0, M) maxima and [M, 2M) minima, with
  // atomicMax -- the range pass of the per-token quantize that follows, done while the values are still in registers.
  uint32_t* row_range;
  // A given as `a_pieces` column blocks of a_piece_cols columns each, block r a row-major [M, a_piece_cols] matrix at
  // A + r * M * a_piece_cols (what an all-gather of column-sharded activations leaves); 1 = plain row-major [M, K].
  int a_pieces;
  int a_piece_cols;
  // Order in which the persistent CTAs walk the tiles.  0: row block by row block (all column tiles of a row block are
  // neighbours).  g > 0: groups of g row blocks, and inside a group column tile by column tile with the group's row
  // blocks as neighbours -- the tiles in flight at one time then share few W tiles, which is what matters when W
  // (N*K bytes) is larger than L2: walked row block by row block, the whole of W streams from HBM once per row block.
  int group_m;
  uint32_t* status;
  unsigned long long wait_limit_ns;
};

// Row-block and column-tile index of tile number `tile` in the walking order above.
__device__ __forceinline__ void tile_coords(const GemmParams& p, int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t& tm, int64_t& tn) {
  if (p.group_m == 0) {
    tm = tile / tiles_n;
    tn = tile - tm * tiles_n;
    return;
  }
  const int64_t per_group = (int64_t)p.group_m * tiles_n;
  const int64_t g = tile / per_group, r = tile - g * per_group;
  const int64_t m_first = g * p.group_m;
  const int64_t gm = (tiles_m - m_first < p.group_m) ? tiles_m - m_first : p.group_m;   // the last group may be smaller
  tn = r / gm;
  tm = m_first + (r - tn * gm);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One probe of the barrier.  The hint lets the hardware park the thread for up to that many nanoseconds while the
// phase is incomplete (it wakes as soon as the phase completes), so a waiting role does not burn the issue slots
// the epilogue warps of its scheduler need.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)
      : "memory");
  return ok != 0;
}
// Bounded wait: false means "give up" (either this wait ran out or another role raised the abort flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 3u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Three-dimensional forms (A stored as column blocks: coordinates are column within the block, row, block).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* tm, uint32_t bar_cluster, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// The same copy issued by a CTA of a pair: the mbarrier may live in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
// Address of `local` (a shared::cta address) in the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 128 B,
// groups of 8 rows 1024 B apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;              // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;    // stride byte offset
  d |= (uint64_t)1 << 46;              // version
  d |= (uint64_t)2 << 61;              // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::i8: D = S32, A = B = signed 8-bit, both K-major, M = 128, N = 256.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
        "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// Waits for the thread's tensor-memory loads.  The loaded registers are in/out operands so that no use of them can
// be scheduled ahead of the wait (the load itself only starts the transfer).
__device__ __forceinline__ void tmem_ld_wait16(int (&v)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]), "+r"(v[8]),
                 "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
               :
               : "memory");
}

// Bulk-tensor store of one staging tile (shared -> global), tracked by the issuing thread's bulk async-group.
// Rows and columns of the box that lie outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(reinterpret_cast<uint64_t>(tm)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Until every store this thread issued has finished READING its staging tile / has completed altogether.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Generic-proxy writes to shared memory become visible to the async proxy (the bulk copy engine).
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

struct alignas(16) Misc {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  union {                                 // one table per kernel variant, by the arithmetic of its sigmoid tail
    float exp_ff[2 * EXP_FF_ENTRIES];       // binary32 pairs (fill_exp_ff_table)
    double exp2[EXP2_TABLE_SIZE];           // binary64 (fill_exp2_table)
  };
  alignas(16) float col_scale[4 * BN];   // per-warp copy of w_scales for the warp's columns of the tile (read as float4)
  alignas(16) float col_bias[4 * BN];
};
static_assert(sizeof(Misc) <= MISC_BYTES, "misc region too small");
static_assert(offsetof(Misc, col_scale) % 16 == 0 && offsetof(Misc, col_bias) % 16 == 0, "float4 reads need 16-byte alignment");

enum OutMode : int { OUT_F32 = 0, OUT_I32 = 1, OUT_Q8 = 2 };

template <int ACT_T, int OUT_T, int NCTA, int EW = 8>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
gemm_i8_umma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using C = Cfg<NCTA, EW>;
  constexpr int STAGES = C::STAGES, STAGE_BYTES = C::STAGE_BYTES, A_BYTES = C::A_BYTES;
  constexpr int EPI_WARPS = EW, EPI_COLS = C::EPI_COLS;
  extern __shared__ uint8_t smem_raw[];
  // The pair variant needs the same shared-memory offsets in both CTAs: the dynamic region starts at the
  // same window offset in every CTA of a kernel, so rounding it up to 1024 B gives the same result in both.
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* out_stage = tiles + STAGES * STAGE_BYTES;   // 1024-byte aligned: EPI_WARPS staging tiles of the epilogue
  Misc* misc = reinterpret_cast<Misc*>(out_stage + EPI_WARPS * OUT_STAGE_BYTES);
  volatile int* abort_flag = &misc->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = NCTA == 2 ? cluster_cta_rank() : 0u;   // 0 = the CTA that issues the MMAs
  // A programmatic dependent of this launch (the next quantize) may take over SMs as this kernel's CTAs leave them.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int64_t tiles_n = (p.N + BN - 1) / BN, tiles_m = (p.M + BM * NCTA - 1) / (BM * NCTA);
  const int64_t num_tiles = tiles_m * tiles_n;
  const int64_t tile_first = blockIdx.x / NCTA, tile_step = gridDim.x / NCTA;
  const int num_kb = (int)((p.K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(smem_u32(&misc->full[s]), 1);
      mbar_init(smem_u32(&misc->empty[s]), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(smem_u32(&misc->tmem_full[s]), 1);
      mbar_init(smem_u32(&misc->tmem_empty[s]), EPI_WARPS * NCTA);  // the epilogue warps of both CTAs of a pair
    }
    misc->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (ACT_T == ACT_GELU_SIGMOID_F32 || ACT_T == ACT_SILU_F32) fill_exp_ff_table(misc->exp_ff, threadIdx.x, blockDim.x);
  else if (ACT_T == ACT_GELU_SIGMOID || ACT_T == ACT_SILU) fill_exp2_table(misc->exp2, threadIdx.x, blockDim.x);
  if (warp == 1) {
    if (NCTA == 1) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&misc->tmem_base)),
                   "r"((uint32_t)TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {  // the same warp of both CTAs allocates, with the same destination offset
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&misc->tmem_base)),
                   "r"((uint32_t)TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
  }
  __syncthreads();
  if (NCTA == 2) cluster_sync_all();  // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  // Launched as a programmatic dependent of the previous kernel of the stream (which usually produced A and its
  // scales), everything above overlaps that kernel's tail; nothing below may run before it has finished.
  // Without that launch attribute this is a no-op.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint32_t tmem_base = misc->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = tile_first; ok && tile < num_tiles; tile += tile_step) {
        int64_t tm, tn;
        tile_coords(p, tile, tiles_m, tiles_n, tm, tn);
        const int m0 = (int)tm * (BM * NCTA) + (int)cta_rank * BM;
        const int n0 = (int)tn * BN + (int)cta_rank * C::B_ROWS;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&misc->empty[s]), ph ^ 1u, abort_flag, p.wait_limit_ns)) {
            atomicOr(p.status, STATUS_TMA_WAIT_TIMEOUT);
            ok = false;
            break;
          }
          const uint32_t bar = smem_u32(&misc->full[s]);
          uint8_t* st = tiles + s * STAGE_BYTES;
          // K block kb of A when A is stored as column blocks: block and column inside it (a block boundary never falls
          // inside a K block: the host requires a_piece_cols to be a multiple of BK)
          const int a_piece = p.a_pieces > 1 ? (kb * BK) / p.a_piece_cols : 0;
          const int a_col = p.a_pieces > 1 ? (kb * BK) - a_piece * p.a_piece_cols : 0;
          if (NCTA == 1) {
            mbar_expect_tx(bar, STAGE_BYTES);
            if (p.a_pieces > 1) tma_load_3d(smem_u32(st), &tmA, bar, a_col, m0, a_piece);
            else tma_load_2d(smem_u32(st), &tmA, bar, kb * BK, m0);
            tma_load_2d(smem_u32(st + A_BYTES), &tmB, bar, kb * BK, n0);
          } else {
            // Both CTAs' copies complete on the barrier of the MMA-issuing CTA, which expects the bytes of both.
            // (A partner's bytes may land before the expectation is posted; the count is signed.)
            if (cta_rank == 0) mbar_expect_tx(bar, 2 * STAGE_BYTES);
            const uint32_t bar0 = map_to_cta(bar, 0);
            if (p.a_pieces > 1) tma_load_3d_pair(smem_u32(st), &tmA, bar0, a_col, m0, a_piece);
            else tma_load_2d_pair(smem_u32(st), &tmA, bar0, kb * BK, m0);
            tma_load_2d_pair(smem_u32(st + A_BYTES), &tmB, bar0, kb * BK, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      constexpr uint32_t idesc = make_idesc(BM * NCTA, BN);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int64_t tile = tile_first; ok && tile < num_tiles; tile += tile_step, tile_it++) {
        const uint32_t slot = tile_it & 1u, tph = (tile_it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&misc->tmem_empty[slot]), tph ^ 1u, abort_flag, p.wait_limit_ns)) {
          atomicOr(p.status, STATUS_MMA_WAIT_TIMEOUT);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + slot * BN;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait(smem_u32(&misc->full[s]), ph, abort_flag, p.wait_limit_ns)) {
            atomicOr(p.status, STATUS_MMA_WAIT_TIMEOUT);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
          const uint64_t da = make_smem_desc(a_addr), db = make_smem_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            // advancing K inside the 128-byte swizzle atom = advancing the start address by 32 B
            const uint64_t dak = da + (uint64_t)(k * (UMMA_K >> 4)), dbk = db + (uint64_t)(k * (UMMA_K >> 4));
            if (NCTA == 1) umma_i8(tmem_d, dak, dbk, idesc, (kb | k) ? 1u : 0u);
            else umma_i8_pair(tmem_d, dak, dbk, idesc, (kb | k) ? 1u : 0u);
          }
          // frees the stage (in both CTAs of a pair) when these MMAs have read it
          if (NCTA == 1) umma_commit(smem_u32(&misc->empty[s]));
          else umma_commit_pair(smem_u32(&misc->empty[s]));
        }
        if (ok) {
          if (NCTA == 1) umma_commit(smem_u32(&misc->tmem_full[slot]));
          else umma_commit_pair(smem_u32(&misc->tmem_full[slot]));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int ew = warp - 2;             // 0 .. EW-1
    const int quarter = warp & 3;        // tensor-memory lanes this warp may read: [32*quarter, 32*quarter+32)
    const int col0 = (ew >> 2) * EPI_COLS;  // first tile column of this warp
    float* cs = misc->col_scale + ew * EPI_COLS;
    float* cb = misc->col_bias + ew * EPI_COLS;
    const bool has_bias = p.bias != nullptr;
    // 16-byte stores need every row segment 16-byte aligned: N a multiple of 4 elements (f32, i32) or of 16 (int8).
    const bool vec_ok = OUT_T == OUT_Q8 ? ((p.N % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.out_q) & 15u) == 0))
                        : OUT_T == OUT_I32 ? ((p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.out_i32) & 15u) == 0))
                                           : ((p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.out_f32) & 15u) == 0));
    // 4-byte outputs leave through this warp's staging tile and a bulk-tensor store: the copy engine writes whole
    // 64-byte row segments and clips at M and N, where a lane writing its own row straight from registers issues
    // 16-byte pieces of 32 different lines per instruction (measured: those stores, not the arithmetic, bounded
    // the epilogue).  The tile is laid out for the tensor map's 64-byte swizzle: the 16-byte piece q of row r sits
    // at piece q ^ ((r >> 1) & 3), which also keeps the eight lanes of a store phase on distinct banks.
    // int8 output uses the same tile as 32 rows x 64 codes: four chunks fill it, then one store writes 64-byte segments.
    const bool bulk_store = p.tma_store != 0;
    bool q8_pending = false;   // warp-uniform: the tile holds chunks that have not been stored yet
    int64_t q8_col = 0;        // first column of the group of four chunks in the tile
    const uint32_t stage_addr = smem_u32(out_stage + ew * OUT_STAGE_BYTES);
    const uint32_t stage_row = stage_addr + (uint32_t)lane * (EPI_CH * 4);
    const uint32_t stage_xor = (uint32_t)((lane >> 1) & 3);
    uint32_t tile_it = 0;
    for (int64_t tile = tile_first; tile < num_tiles; tile += tile_step, tile_it++) {
      const uint32_t slot = tile_it & 1u, tph = (tile_it >> 1) & 1u;
      int64_t tm, tn;
      tile_coords(p, tile, tiles_m, tiles_n, tm, tn);
      const int64_t m0 = tm * (BM * NCTA) + cta_rank * BM, n0 = tn * BN + col0;
      if (OUT_T != OUT_I32) {
        // Stage this warp's column scales and biases while the main loop of the tile still runs.
        __syncwarp();
#pragma unroll
        for (int j = lane; j < EPI_COLS; j += 32) {
          const int64_t n = n0 + j;
          cs[j] = (n < p.N) ? __ldg(p.w_scales + n) : 0.0f;
          cb[j] = (has_bias && n < p.N) ? __ldg(p.bias + n) : -0.0f;  // x + (-0) == x for every x, -0 included
        }
        __syncwarp();
      }
      const int64_t mw = m0 + quarter * 32;   // first row of this warp
      const int64_t m = mw + lane;
      const bool row_ok = m < p.M;
      const float a_scale = (p.a_scales && row_ok) ? __ldg(p.a_scales + m) : 1.0f;  // fround(1 * ws) == ws
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(smem_u32(&misc->tmem_full[slot]), tph, abort_flag, p.wait_limit_ns);
        if (!ok) atomicOr(p.status, STATUS_EPI_WAIT_TIMEOUT);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + slot * BN + (uint32_t)col0 + ((uint32_t)(quarter * 32) << 16);
      constexpr int NCH = EPI_COLS / EPI_CH;
      // The accumulator columns of the next chunk travel from tensor memory while the current chunk is computed.
      int a_next[EPI_CH];
      if (n0 < p.N) tmem_ld16(taddr, a_next);
      // running range of this lane's row over the warp's columns of the tile (fminf / fmaxf drop NaN operands)
      const bool want_range = OUT_T == OUT_F32 && p.row_range != nullptr;
      float r_mn = __int_as_float(0x7f800000), r_mx = __int_as_float(0xff800000);
#pragma unroll 1
      for (int c = 0; c < NCH; c++) {
        const int64_t nb = n0 + c * EPI_CH;
        if (nb >= p.N) break;  // uniform across the warp
        int a[EPI_CH];
        tmem_ld_wait16(a_next);
#pragma unroll
        for (int j = 0; j < EPI_CH; j++) a[j] = a_next[j];
        if (c + 1 < NCH && nb + EPI_CH < p.N) tmem_ld16(taddr + (uint32_t)((c + 1) * EPI_CH), a_next);
        // No lane may leave this iteration early: the tensor-memory loads, the votes and the staging protocol below
        // are warp-collective.  Rows past M compute on whatever the accumulator holds and store nothing.
        const bool full = vec_ok && (nb + EPI_CH <= p.N);
        uint32_t v[EPI_CH];   // the chunk's 4-byte results as bit patterns (f32 or i32 output)
        float y[EPI_CH];
        if (OUT_T == OUT_I32) {
#pragma unroll
          for (int j = 0; j < EPI_CH; j++) v[j] = (uint32_t)a[j];
        } else {
          // An accumulator of 2^22 or more anywhere in the warp's chunk sends the whole chunk through the binary64
          // product (the cheap int -> float conversion and the binary32 product are only exact below that).
          bool wide = false;
          if (p.acc_class == 2) {
            int big = 0;
#pragma unroll
            for (int j = 0; j < EPI_CH; j++) big |= (abs(a[j]) >> 22);
            wide = __any_sync(0xffffffffu, big != 0);
          }
          const float4* cs4 = reinterpret_cast<const float4*>(cs + c * EPI_CH);
          const float4* cb4 = reinterpret_cast<const float4*>(cb + c * EPI_CH);
          // The loops below contain no branch at all (the choice between the two conversions is made once per
          // chunk, a missing bias was staged as -0.0, which is the identity of the rounded addition), so the
          // independent element chains of a thread can be interleaved freely.
          if (p.acc_class == 1) {
#pragma unroll
            for (int j4 = 0; j4 < EPI_CH / 4; j4++) {
              const float4 w4 = cs4[j4], b4 = cb4[j4];
              const float wsv[4] = {w4.x, w4.y, w4.z, w4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
              for (int e = 0; e < 4; e++)
                y[j4 * 4 + e] = __fadd_rn(__fmul_rn(__int2float_rn(a[j4 * 4 + e]), __fmul_rn(a_scale, wsv[e])), bv[e]);
            }
          } else if (!wide) {
#pragma unroll
            for (int j4 = 0; j4 < EPI_CH / 4; j4++) {
              const float4 w4 = cs4[j4], b4 = cb4[j4];
              const float wsv[4] = {w4.x, w4.y, w4.z, w4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
              for (int e = 0; e < 4; e++) y[j4 * 4 + e] = __fadd_rn(scale_acc_small(a[j4 * 4 + e], __fmul_rn(a_scale, wsv[e])), bv[e]);
            }
          } else {
#pragma unroll
            for (int j4 = 0; j4 < EPI_CH / 4; j4++) {
              const float4 w4 = cs4[j4], b4 = cb4[j4];
              const float wsv[4] = {w4.x, w4.y, w4.z, w4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
              for (int e = 0; e < 4; e++) y[j4 * 4 + e] = __fadd_rn(scale_acc_wide(a[j4 * 4 + e], __fmul_rn(a_scale, wsv[e])), bv[e]);
            }
          }
          if (ACT_T == ACT_GELU_SIGMOID || ACT_T == ACT_SILU || ACT_T == ACT_GELU_SIGMOID_F32 || ACT_T == ACT_SILU_F32) {
#pragma unroll
            for (int j0 = 0; j0 < EPI_CH; j0 += 8) {
              float r8[8];
#pragma unroll
              for (int e = 0; e < 8; e++) r8[e] = y[j0 + e];
              if (ACT_T == ACT_GELU_SIGMOID || ACT_T == ACT_SILU) apply_sigmoid_act_x8<ACT_T>(r8, misc->exp2);
              else apply_sigmoid_act_wide<ACT_T == ACT_SILU_F32 ? ACT_SILU : ACT_GELU_SIGMOID, 8>(r8, misc->exp_ff);
#pragma unroll
              for (int e = 0; e < 8; e++) y[j0 + e] = r8[e];
            }
          } else if (ACT_T != ACT_NONE) {
#pragma unroll
            for (int j = 0; j < EPI_CH; j++) y[j] = apply_act_fast<ACT_T>(y[j], nullptr);
          }
#pragma unroll
          for (int j = 0; j < EPI_CH; j++) v[j] = __float_as_uint(y[j]);
          if (want_range) {
            if (nb + EPI_CH <= p.N) {
#pragma unroll
              for (int j = 0; j < EPI_CH; j++) { r_mn = fminf(r_mn, y[j]); r_mx = fmaxf(r_mx, y[j]); }
            } else {
#pragma unroll
              for (int j = 0; j < EPI_CH; j++)
                if (nb + j < p.N) { r_mn = fminf(r_mn, y[j]); r_mx = fmaxf(r_mx, y[j]); }
            }
          }
        }
        if (OUT_T != OUT_Q8) {
          if (bulk_store) {
            // The previous store of this warp must have finished reading the tile before it is overwritten.
            if (lane == 0) tma_store_wait_read();
            __syncwarp();
#pragma unroll
            for (int q = 0; q < EPI_CH / 4; q++) {
              const uint32_t dst = stage_row + ((((uint32_t)q) ^ stage_xor) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[q * 4]), "r"(v[q * 4 + 1]), "r"(v[q * 4 + 2]),
                           "r"(v[q * 4 + 3])
                           : "memory");
            }
            fence_async_shared();
            __syncwarp();
            if (lane == 0 && mw < p.M) tma_store_2d(&tmC, stage_addr, (int)nb, (int)mw);
          } else {
            uint32_t* o = (OUT_T == OUT_I32 ? reinterpret_cast<uint32_t*>(p.out_i32) : reinterpret_cast<uint32_t*>(p.out_f32)) + m * p.N + nb;
            if (!row_ok) {
            } else if (full) {
#pragma unroll
              for (int j = 0; j < EPI_CH; j += 4) *reinterpret_cast<uint4*>(o + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < EPI_CH; j++)
                if (nb + j < p.N) o[j] = v[j];
            }
          }
        } else {
          int8_t* o = p.out_q + m * p.N + nb;
          uint32_t words[EPI_CH / 4];
          QuantGuard guard;
#pragma unroll
          for (int j4 = 0; j4 < EPI_CH / 4; j4++)
            words[j4] = pack_codes(quantize_fast(y[j4 * 4 + 0], p.q_inv, guard), quantize_fast(y[j4 * 4 + 1], p.q_inv, guard),
                                   quantize_fast(y[j4 * 4 + 2], p.q_inv, guard), quantize_fast(y[j4 * 4 + 3], p.q_inv, guard));
          if (p.q_exact || guard.unsafe(127.49f)) {  // rare: a tie, a value beyond the clamp, NaN
#pragma unroll
            for (int j4 = 0; j4 < EPI_CH / 4; j4++)
              words[j4] = pack_codes(quantize_exact_c(y[j4 * 4 + 0], p.q_scale, 0.0f, -128.0f, 127.0f),
                                     quantize_exact_c(y[j4 * 4 + 1], p.q_scale, 0.0f, -128.0f, 127.0f),
                                     quantize_exact_c(y[j4 * 4 + 2], p.q_scale, 0.0f, -128.0f, 127.0f),
                                     quantize_exact_c(y[j4 * 4 + 3], p.q_scale, 0.0f, -128.0f, 127.0f));
          }
          static_assert(EPI_CH == 16, "one 16-byte piece per row and chunk");
          if (bulk_store) {
            const uint32_t piece = (uint32_t)(c & 3);
            if (piece == 0) {  // a new group: the store of the previous one must have read the tile
              if (lane == 0) tma_store_wait_read();
              __syncwarp();
              q8_col = nb;
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_row + ((piece ^ stage_xor) << 4)), "r"(words[0]),
                         "r"(words[1]), "r"(words[2]), "r"(words[3])
                         : "memory");
            q8_pending = true;
            if (piece == 3) {
              fence_async_shared();
              __syncwarp();
              if (lane == 0 && mw < p.M) tma_store_2d(&tmC, stage_addr, (int)q8_col, (int)mw);
              q8_pending = false;
            }
          } else if (!row_ok) {
          } else if (full) {
            *reinterpret_cast<uint4*>(o) = make_uint4(words[0], words[1], words[2], words[3]);
          } else {
#pragma unroll
            for (int j = 0; j < EPI_CH; j++)
              if (nb + j < p.N) o[j] = (int8_t)((words[j >> 2] >> (8 * (j & 3))) & 0xff);
          }
        }
      }
      if (want_range && row_ok) {   // +Inf / -Inf left in place mean "nothing but NaN seen": nothing to publish
        if (r_mx != __int_as_float(0xff800000)) atomicMax(p.row_range + m, range_key_max(r_mx));
        if (r_mn != __int_as_float(0x7f800000)) atomicMax(p.row_range + p.M + m, range_key_min(r_mn));
      }
      if (OUT_T == OUT_Q8 && q8_pending) {  // N ended inside a group of four chunks: columns past N are clipped
        fence_async_shared();
        __syncwarp();
        if (lane == 0 && mw < p.M) tma_store_2d(&tmC, stage_addr, (int)q8_col, (int)mw);
        q8_pending = false;
      }
      // this warp is done reading the accumulator: hand the slot back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (NCTA == 1) mbar_arrive(smem_u32(&misc->tmem_empty[slot]));
        else mbar_arrive_cluster(map_to_cta(smem_u32(&misc->tmem_empty[slot]), 0));
      }
    }
    // Bulk stores still in flight read this CTA's shared memory: they finish before the CTA may leave.
    if (bulk_store && lane == 0) tma_store_wait_all();
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    // Something gave up.  Let bulk copies and MMAs that are still in flight finish
    // before shared and tensor memory are released (bounded: 2 ms).
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (NCTA == 2) cluster_sync_all();  // neither CTA leaves while its partner may still signal its barriers or read its tiles
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    if (NCTA == 1)
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
  }
}

// The give-up path of mbar_wait on a healthy device: a barrier in shared memory that expects one arrival and never
// gets it, nothing asynchronous in flight.  The wait must return false after limit_ns.
__global__ void selftest_bounded_wait_kernel(uint32_t* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  abort_word = 0;
  mbar_init(smem_u32(&bar), 1);
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  volatile int* abort_flag = &abort_word;
  if (!mbar_wait(smem_u32(&bar), 0u, abort_flag, limit_ns) && *abort_flag) atomicOr(status, STATUS_SELFTEST_WAIT_TIMEOUT);
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&bar)) : "memory");
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Row-major int8 matrix [rows, K]; box = 128 bytes of K by box_rows rows, 128-byte swizzle, zero fill outside.
int make_tensor_map(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t K, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  B200Q_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200Q_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (rows=%lld K=%lld)", (int)r, (long long)rows,
                (long long)K);
  return 0;
}

// int8 matrix stored as `pieces` column blocks, block r a row-major [rows, piece_cols] matrix at ptr + r * rows * piece_cols:
// a three-dimensional map (column in block, row, block) with the same box as make_tensor_map, so a K block lands in
// shared memory exactly as it would from a row-major matrix.
int make_tensor_map_pieces(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t piece_cols, int pieces, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  B200Q_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[3] = {(cuuint64_t)piece_cols, (cuuint64_t)rows, (cuuint64_t)pieces};
  cuuint64_t gstride[2] = {(cuuint64_t)piece_cols, (cuuint64_t)piece_cols * (cuuint64_t)rows};
  cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200Q_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (rows=%lld piece_cols=%lld pieces=%d)", (int)r,
                (long long)rows, (long long)piece_cols, pieces);
  return 0;
}

// Row-major output [M, N]; the box is what one epilogue warp stores at a time: 32 rows by 64 bytes (EPI_CH 4-byte
// values, or 64 int8 codes), 64-byte swizzle.
int make_output_map(CUtensorMap* tm, void* ptr, int64_t M, int64_t N, CUtensorMapDataType dtype, int elem_bytes) {
  EncodeTiledFn enc = get_encode_fn();
  B200Q_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[2] = {(cuuint64_t)N, (cuuint64_t)M};
  cuuint64_t gstride[1] = {(cuuint64_t)N * (cuuint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(64 / elem_bytes), 32};
  cuuint32_t estr[2] = {1, 1};
  static_assert(EPI_CH * 4 == 64, "the staging tile is laid out for the 64-byte swizzle");
  CUresult r = enc(tm, dtype, 2, ptr, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B200Q_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (output M=%lld N=%lld)", (int)r, (long long)M,
                (long long)N);
  return 0;
}

}  // namespace

int launch_selftest_bounded_wait(b200q_ctx* ctx, unsigned long long limit_ns) {
  selftest_bounded_wait_kernel<<<1, 1, 0, ctx->stream>>>(ctx->status_dev, limit_ns);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

bool gemm_umma_supported(const void* A, const void* W, int64_t M, int64_t N, int64_t K) {
  return M > 0 && N > 0 && K > 0 && (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15u) == 0) &&
         ((reinterpret_cast<uintptr_t>(W) & 15u) == 0) && M < (1ll << 31) - BM && N < (1ll << 31) - BN && K < (1ll << 31) - BK;
}

int launch_gemm_i8_umma(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K,
                        const float* a_scales, const float* w_scales, const float* bias, int act, float* out_f32,
                        int32_t* out_i32, int8_t* out_q, double q_scale, uint32_t* row_range, int a_pieces) {
  ProfScope prof(ctx, KK_GEMM_UMMA);
  B200Q_REQUIRE(a_pieces >= 1, "tensor-core int8 gemm: the activations are stored as at least one column block");
  B200Q_REQUIRE(a_pieces == 1 || (K % a_pieces == 0 && (K / a_pieces) % BK == 0),
                "tensor-core int8 gemm: column blocks of the activations must be equal and a multiple of %d columns wide (K=%lld in %d blocks)",
                BK, (long long)K, a_pieces);
  B200Q_REQUIRE(row_range == nullptr || out_f32 != nullptr, "tensor-core int8 gemm: row ranges are published with f32 output only");
  // The launch may begin while the previous kernel of the stream drains (programmatic dependent launch): the set-up
  // of this kernel overlaps that tail, and its griddepcontrol.wait holds everything else back until the previous
  // kernel -- whatever it was -- has completed.  With profiling on an event sits between the two anyway.
  const bool after_producer = !ctx->profiling;
  B200Q_REQUIRE(gemm_umma_supported(A, W_nk, M, N, K), "tensor-core int8 gemm needs K %% 16 == 0 and 16-byte aligned operands");
  // CTA pairs pay off once there are enough 256-row tiles to go round; small or forced cases use single CTAs.
  const int ncta = ctx->gemm_variant == 2 ? 1 : ctx->gemm_variant == 3 ? 2 : (M >= 1024 ? 2 : 1);
  CUtensorMap tmA, tmB, tmC;
  if (a_pieces > 1) {
    if (int e = make_tensor_map_pieces(&tmA, A, M, K / a_pieces, a_pieces, BM)) return e;
  } else if (int e = make_tensor_map(&tmA, A, M, K, BM)) return e;
  if (int e = make_tensor_map(&tmB, W_nk, N, K, BN / ncta)) return e;
  GemmParams p;
  // Bulk-tensor stores need a 16-byte aligned base and row pitch.
  void* out_any = out_f32 ? static_cast<void*>(out_f32) : out_i32 ? static_cast<void*>(out_i32) : static_cast<void*>(out_q);
  const int out_elem = out_q ? 1 : 4;
  p.tma_store = out_any != nullptr && (N * out_elem) % 16 == 0 && (reinterpret_cast<uintptr_t>(out_any) & 15u) == 0;
  if (p.tma_store) {
    const CUtensorMapDataType dt = out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : out_i32 ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    if (int e = make_output_map(&tmC, out_any, M, N, dt, out_elem)) return e;
  } else {
    memset(&tmC, 0, sizeof(tmC));   // never dereferenced
  }
  p.M = M; p.N = N; p.K = K;
  p.a_scales = a_scales; p.w_scales = w_scales; p.bias = bias; p.act = act;
  p.out_f32 = out_f32; p.out_i32 = out_i32; p.out_q = out_q;
  p.q_scale = q_scale;
  p.row_range = row_range;
  p.acc_class = K <= 255 ? 0 : K <= 1024 ? 1 : 2;
  p.a_pieces = a_pieces;
  p.a_piece_cols = (int)(K / a_pieces);
  {
    // Walking order of the tiles: grouped when W is too large to stay in L2 (126 MB) next to the rest -- all row blocks
    // in one group when A is small enough to stay resident beside the W tiles in flight, groups of 8 otherwise (the
    // tiles in flight then touch about 8 row blocks and 9 column tiles: the smallest footprint a wave of 74 can have).
    const int64_t tiles_m = (M + (int64_t)BM * ncta - 1) / ((int64_t)BM * ncta);
    int g = ctx->tile_group;
    if (g < 0) g = (N * K > (int64_t(48) << 20) && tiles_m > 1) ? (M * K <= (int64_t(48) << 20) ? (int)tiles_m : 8) : 0;
    if (g > tiles_m) g = (int)tiles_m;
    p.group_m = g;
  }
  p.q_inv = 0.0f; p.q_exact = 0;
  if (out_q) {
    p.q_inv = (float)(1.0 / q_scale);
    float a = p.q_inv < 0 ? -p.q_inv : p.q_inv;
    p.q_exact = !(a >= 1.17549435e-38f && a <= 3.402823466e38f);
  }
  p.status = ctx->status_dev;
  p.wait_limit_ns = (unsigned long long)(ctx->wait_limit_s * 1e9);
  const int64_t num_tiles = ((M + BM * ncta - 1) / (BM * ncta)) * ((N + BN - 1) / BN);
  const int64_t units = ctx->sm_count / ncta;   // CTAs (or CTA pairs) that can be resident at once
  const unsigned grid = (unsigned)((num_tiles < units ? num_tiles : units) * ncta);
  typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const GemmParams);
#define B200Q_ROW(A) \
  {{gemm_i8_umma_kernel<A, OUT_F32, 1>, gemm_i8_umma_kernel<A, OUT_F32, 2>}, {gemm_i8_umma_kernel<A, OUT_Q8, 1>, gemm_i8_umma_kernel<A, OUT_Q8, 2>}}
  static const KernelFn table[5][2][2] = {B200Q_ROW(ACT_NONE), B200Q_ROW(ACT_RELU), B200Q_ROW(ACT_GELU_SIGMOID),
                                          B200Q_ROW(ACT_GELU_TANH), B200Q_ROW(ACT_SILU)};
#undef B200Q_ROW
  static const KernelFn raw[2] = {gemm_i8_umma_kernel<ACT_NONE, OUT_I32, 1>, gemm_i8_umma_kernel<ACT_NONE, OUT_I32, 2>};
  // f32 output with the approximate sigmoid tails (b200q_set_tail_mode 1): [gelu_sigmoid, silu][CTAs per tile]
  static const KernelFn approx[2][2] = {{gemm_i8_umma_kernel<ACT_GELU_SIGMOID_APPROX, OUT_F32, 1>, gemm_i8_umma_kernel<ACT_GELU_SIGMOID_APPROX, OUT_F32, 2>},
                                        {gemm_i8_umma_kernel<ACT_SILU_APPROX, OUT_F32, 1>, gemm_i8_umma_kernel<ACT_SILU_APPROX, OUT_F32, 2>}};
  // The same exact values from binary32 arithmetic alone, for launches whose main loop keeps the tensor pipe busy for
  // longer than the tail takes: binary64 instructions slow down several times while MMAs are in flight (C3 and
  // C5 shapes gain 3 to 5 %), but run on an otherwise idle pipe when the tail is the longer part (K 768: 172 us
  // against 203 us).
  static const KernelFn tensor_bound[2][2] = {{gemm_i8_umma_kernel<ACT_GELU_SIGMOID_F32, OUT_F32, 1>, gemm_i8_umma_kernel<ACT_GELU_SIGMOID_F32, OUT_F32, 2>},
                                              {gemm_i8_umma_kernel<ACT_SILU_F32, OUT_F32, 1>, gemm_i8_umma_kernel<ACT_SILU_F32, OUT_F32, 2>}};
  // Sixteen epilogue warps for f32 output when the main loop of a tile is short (K up to 1024): [activation][CTAs per tile]
#define B200Q_WIDE(A) {gemm_i8_umma_kernel<A, OUT_F32, 1, 16>, gemm_i8_umma_kernel<A, OUT_F32, 2, 16>}
  static const KernelFn wide[5][2] = {B200Q_WIDE(ACT_NONE), B200Q_WIDE(ACT_RELU), B200Q_WIDE(ACT_GELU_SIGMOID), B200Q_WIDE(ACT_GELU_TANH),
                                      B200Q_WIDE(ACT_SILU)};
#undef B200Q_WIDE
  constexpr int64_t WIDE_EPILOGUE_MAX_K = 1024;
  constexpr int64_t SIGMOID_F32_MIN_K = 4096;
  B200Q_REQUIRE(act >= 0 && act <= 4, "unknown activation %d", act);
  B200Q_REQUIRE((out_i32 != nullptr) + (out_f32 != nullptr) + (out_q != nullptr) == 1,
                "tensor-core int8 gemm writes exactly one output");
  KernelFn fn = out_i32 ? raw[ncta - 1] : table[act][out_q ? 1 : 0][ncta - 1];
  int slot_act = act;
  if (out_f32 != nullptr && (act == ACT_GELU_SIGMOID || act == ACT_SILU)) {
    if (ctx->tail_mode == 1) {
      fn = approx[act == ACT_SILU ? 1 : 0][ncta - 1];
      slot_act = act == ACT_SILU ? 6 : 5;
    } else if (K >= SIGMOID_F32_MIN_K) {
      fn = tensor_bound[act == ACT_SILU ? 1 : 0][ncta - 1];
      slot_act = act == ACT_SILU ? 8 : 7;
    }
  }
  int epi_warps = 8;
  // Measured at M 16384, K 768: the exact sigmoid tails gain 9 % from sixteen warps (168 -> 153 us at N 3072), the
  // short tails gain nothing (52 us either way at N 2304: their pace is set by the stores), so only the former switch.
  const bool long_tail = act == ACT_GELU_SIGMOID || act == ACT_SILU;
  if (out_f32 != nullptr && fn == table[act][0][ncta - 1] && ctx->epilogue_warps != 8 &&
      (ctx->epilogue_warps == 16 || (K <= WIDE_EPILOGUE_MAX_K && long_tail))) {
    fn = wide[act][ncta - 1];
    slot_act = 9 + act;
    epi_warps = 16;
  }
  const int smem = epi_warps == 16 ? (ncta == 1 ? smem_bytes<1, 16>() : smem_bytes<2, 16>()) : (ncta == 1 ? smem_bytes<1>() : smem_bytes<2>());
  const int slot_idx = (out_i32 ? 31 : slot_act * 2 + (out_q ? 1 : 0)) * 2 + (ncta - 1);   // < 64
  if (!(ctx->umma_ready_mask & (1ull << slot_idx))) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    ctx->umma_ready_mask |= 1ull << slot_idx;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(64 + 32 * epi_warps);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ncta;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (after_producer) {   // may start while the previous kernel of the stream drains (see griddepcontrol.wait in the kernel)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  B200Q_CHECK_CUDA(cudaLaunchKernelEx(&cfg, fn, tmA, tmB, tmC, p));
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200q
