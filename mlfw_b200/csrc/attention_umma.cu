// softmax(q k^T * scale + mask) v in binary32 accuracy on the 5th-generation tensor cores.
//
// Reference semantics: scaled_dot_product_attention (src/nn/functional/attention.ts:42-74) with the decomposed
// softmax (src/compiler/passes/decompose/decomposition_pass.ts:156-174), every operation in binary32.  The bar is
// 1e-5 of the output's largest magnitude, which one tf32 product (2^-11) misses; each product is therefore taken
// three ways, a = a_hi + a_lo with a_hi the value rounded to tf32 and a_lo the exact remainder:
//     a b  ~  a_hi b_hi + a_hi b_lo + a_lo b_hi            (the dropped a_lo b_lo is below 2^-22 of the product)
// with tcgen05.mma.kind::tf32 and binary32 accumulation in tensor memory.
//
// One CTA of 256 threads per (batch, head, block of 128 queries): query row r (tensor-memory lane r) is shared by the
// two threads r and r + 128, which take the lower and the upper half of every row of scores and of outputs (warps w
// and w + 4 reach the same 32 lanes of tensor memory).  They agree on the row's running maximum through shared memory
// once per step and keep a partial sum each.
// Two CTAs share an SM (96 KB of shared memory and 256 columns of tensor memory each): every phase of a step waits
// on the one before it, so a single CTA leaves the tensor cores, the load path and the arithmetic units idle in turn,
// and the second CTA fills those gaps.  Q_hi lives in shared memory, Q_lo in tensor memory (the A operand of an MMA may
// come from either).  Per step of 64 keys:
//   the threads read the K and V rows from global memory (L2 after the first query block of a head) and split them into
//   hi / lo tiles in the tensor cores' K-major, 128-byte-swizzled layout (V transposed on the way: its tile is
//   [head dim][keys], keys contiguous) -- V while the step's S = Q K^T is on the tensor cores, the next step's K while
//   its P V is;
//   one thread issues S = Q K^T (24 MMAs of 128 x 64 x 8) into tensor memory;
//   every thread reads its half row of S, scales and masks it, keeps the running maximum and sum (online softmax) and
//   writes p = exp2(...) back to tensor memory as P_hi (over S, which is in registers by then) and P_lo;
//   one thread issues O_step = P V (24 MMAs, the A operand read from tensor memory);
//   every thread reads its half row of O_step and folds it into its 32 output registers: o = o * alpha + O_step.
// At the end o / sum goes to global memory.  Queries or keys beyond S read as zeros and are masked / not stored.
//
// Every wait is bounded; a wait that runs out sets STATUS_SDPA_WAIT_TIMEOUT, all threads of the CTA agree to stop
// (a block-wide vote after every wait), let the tensor cores drain for 2 ms, free tensor memory and return.
#include <cuda.h>

#include "common.cuh"
#include "kernels.cuh"

namespace b200q {

namespace {

constexpr int QB = 128, KB = 64, DH = 64, THREADS = 256, HALF = 32;
constexpr int Q_TILE = 2 * QB * 128;                 // two K blocks (32 floats each) of [128 rows][128 B]
constexpr int K_TILE = 2 * KB * 128;
// K: per K block one tile of 128 rows, K_hi in rows 0..63 and K_lo in rows 64..127, so that one MMA of N = 128 takes both
constexpr int SM_QHI = 0, SM_K = Q_TILE, SM_VHI = SM_K + 2 * K_TILE, SM_VLO = SM_VHI + K_TILE, SM_END = SM_VLO + K_TILE;
constexpr int SDPA_SMEM = SM_END + 1024;             // 97 KB + slack to align the tiles to 1024 B: two CTAs per SM
// tensor memory columns: the scores and, once they are in registers, P_hi in their place; P_lo; the step's P V; Q_lo
constexpr int TM_S = 0, TM_S2 = 64, TM_PHI = 0, TM_PLO = 64, TM_O = 128, TM_QLO = 192, TM_COLS = 256;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t gtimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Byte offset of (row, byte column) inside a [rows][128 B] tile with the 128-byte swizzle (16-byte chunks XOR row % 8).
__device__ __forceinline__ uint32_t sw128(int row, int byte_col) {
  return (uint32_t)(row * 128 + ((((byte_col >> 4) ^ (row & 7)) << 4) | (byte_col & 15)));
}
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {   // K-major, 128-byte swizzle, 8-row groups 1024 B apart
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::tf32: D = F32 (1), A = B = TF32 (2), both K-major.
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
      "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d),
      "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
// 32 consecutive columns of this warp's lanes.
__device__ __forceinline__ void ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
      "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
        "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  // the load only starts the transfer: tie every loaded register to a statement after the wait, so that no use of
  // them can be scheduled ahead of it
#pragma unroll
  for (int h = 0; h < 2; h++)
    asm volatile("" : "+r"(r[h * 16 + 0]), "+r"(r[h * 16 + 1]), "+r"(r[h * 16 + 2]), "+r"(r[h * 16 + 3]), "+r"(r[h * 16 + 4]), "+r"(r[h * 16 + 5]),
                      "+r"(r[h * 16 + 6]), "+r"(r[h * 16 + 7]), "+r"(r[h * 16 + 8]), "+r"(r[h * 16 + 9]), "+r"(r[h * 16 + 10]),
                      "+r"(r[h * 16 + 11]), "+r"(r[h * 16 + 12]), "+r"(r[h * 16 + 13]), "+r"(r[h * 16 + 14]), "+r"(r[h * 16 + 15])
                 :
                 : "memory");
#pragma unroll
  for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ uint32_t tf32_rna(float x) {   // nearest tf32 (ties away), low 13 bits zero
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void split4(const float4& v, uint4& hi, uint4& lo) {
  hi.x = tf32_rna(v.x); hi.y = tf32_rna(v.y); hi.z = tf32_rna(v.z); hi.w = tf32_rna(v.w);
  lo.x = __float_as_uint(__fsub_rn(v.x, __uint_as_float(hi.x))); lo.y = __float_as_uint(__fsub_rn(v.y, __uint_as_float(hi.y)));
  lo.z = __float_as_uint(__fsub_rn(v.z, __uint_as_float(hi.z))); lo.w = __float_as_uint(__fsub_rn(v.w, __uint_as_float(hi.w)));
}
// Barrier of the two warps that share a quarter of the lanes (immediate barrier numbers: a register operand would
// reserve all sixteen barriers of the SM for one CTA).
__device__ __forceinline__ void pair_barrier(int quarter) {
  switch (quarter) {
    case 0: asm volatile("bar.sync 1, 64;" ::: "memory"); break;
    case 1: asm volatile("bar.sync 2, 64;" ::: "memory"); break;
    case 2: asm volatile("bar.sync 3, 64;" ::: "memory"); break;
    default: asm volatile("bar.sync 4, 64;" ::: "memory"); break;
  }
}
struct SdpaParams {
  const float *q, *k, *v;
  float* out;
  int64_t ld_q, ld_k, ld_v, ld_o;
  int H, S, q_blocks;
  float scale_log2e;       // scale * log2(e): scores are kept in units of log2
  int causal;
  uint32_t* status;
  unsigned long long limit_ns;
};

__global__ void __launch_bounds__(THREADS, 2) sdpa_umma_kernel(const SdpaParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ float row_xchg[2][QB];   // [half][row]: a step's maximum, at the end the sum, of that half of the row
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sm_base = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // heaviest query blocks (most keys under the causal mask) first
  const int qb = p.q_blocks - 1 - (int)(blockIdx.x % p.q_blocks);
  const int bh = (int)(blockIdx.x / p.q_blocks);
  const int b = bh / p.H, h = bh - b * p.H;
  const int q0 = qb * QB;
  const int kv_end = p.causal ? min(p.S, q0 + QB) : p.S;        // keys this block can see
  const int steps = (kv_end + KB - 1) / KB;
  const float* qg = p.q + ((int64_t)b * p.S) * p.ld_q + (int64_t)h * DH;
  const float* kg = p.k + ((int64_t)b * p.S) * p.ld_k + (int64_t)h * DH;
  const float* vg = p.v + ((int64_t)b * p.S) * p.ld_v + (int64_t)h * DH;

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&bar)), "r"(1) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)TM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    fence_before();
  }

  __syncthreads();
  fence_after();
  const uint32_t tmem = tmem_slot;
  const int half = warp >> 2, row = tid & (QB - 1);                      // which half of the row; the row inside the block
  const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);  // this warp's 32 lanes of tensor memory
  const int qi = q0 + row;                       // this thread's query
  // Q: thread t takes row t: hi to the shared-memory tile (two K blocks of 32 head-dim values), lo to tensor memory
  {
    const float4* src = reinterpret_cast<const float4*>(qg + (int64_t)qi * p.ld_q);
#pragma unroll
    for (int c = 2 * half; c < 2 * half + 2; c++) {
      uint32_t lo16[16];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int d4 = c * 4 + i;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (qi < p.S) x = __ldg(src + d4);
        uint4 hi, lo;
        split4(x, hi, lo);
        *reinterpret_cast<uint4*>(sm + SM_QHI + (uint32_t)((d4 >> 3) * (QB * 128)) + sw128(row, (d4 & 7) * 16)) = hi;
        lo16[4 * i] = lo.x; lo16[4 * i + 1] = lo.y; lo16[4 * i + 2] = lo.z; lo16[4 * i + 3] = lo.w;
      }
      st16(lane_addr + TM_QLO + c * 16, lo16);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }

  const uint32_t bar_addr = smem_u32(&bar);
  uint32_t phase = 0;

  float o[HALF];
#pragma unroll
  for (int d = 0; d < HALF; d++) o[d] = 0.0f;
  float m_run = __int_as_float(0xff800000), l_run = 0.0f;
  bool alive = true;

  auto wait_mma = [&]() -> bool {
    bool ok = true;
    uint32_t done = 0;
    const uint64_t t0 = gtimer();
    uint32_t it = 0;
    while (true) {
      asm volatile(
          "{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, q;\n\t}"
          : "=r"(done)
          : "r"(bar_addr), "r"(phase), "r"(1000u)
          : "memory");
      if (done) break;
      if ((++it & 7u) == 0u && gtimer() - t0 > p.limit_ns) { ok = false; break; }
    }
    phase ^= 1u;
    return __syncthreads_and(ok ? 1 : 0) != 0;     // all threads take the same way out
  };

  // K of the step that starts at key0: global -> hi / lo tiles, row = key (16 consecutive threads read one row's 256 bytes)
  auto stage_k = [&](int key0) {
    float4 x[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int c = i * THREADS + tid, kr = c >> 4, d4 = c & 15;
      x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (key0 + kr < p.S) x[i] = __ldg(reinterpret_cast<const float4*>(kg + (int64_t)(key0 + kr) * p.ld_k) + d4);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int c = i * THREADS + tid, kr = c >> 4, d4 = c & 15;
      uint4 hi, lo;
      split4(x[i], hi, lo);
      const uint32_t off = (uint32_t)((d4 >> 3) * (2 * KB * 128)) + sw128(kr, (d4 & 7) * 16);
      *reinterpret_cast<uint4*>(sm + SM_K + off) = hi;
      *reinterpret_cast<uint4*>(sm + SM_K + off + KB * 128) = lo;
    }
  };
  // V of that step: global -> transposed hi / lo tiles, row = head-dim index, columns = keys (lane = key inside a block
  // of 32, so a warp writes whole 128-byte tile rows; the eight warps take neighbouring 16-byte pieces of the same key's row)
  auto stage_v = [&](int key0) {
    float4 x[4];
#pragma unroll
    for (int kb = 0; kb < 2; kb++)
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int d4 = warp + 8 * i, key = key0 + kb * 32 + lane;
        x[kb * 2 + i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (key < p.S) x[kb * 2 + i] = __ldg(reinterpret_cast<const float4*>(vg + (int64_t)key * p.ld_v) + d4);
      }
#pragma unroll
    for (int kb = 0; kb < 2; kb++)
#pragma unroll
      for (int i = 0; i < 2; i++) {
        const int d4 = warp + 8 * i;
        uint4 hi, lo;
        split4(x[kb * 2 + i], hi, lo);
        const uint32_t tile = (uint32_t)(kb * (KB * 128));
        const uint32_t hv[4] = {hi.x, hi.y, hi.z, hi.w}, lv[4] = {lo.x, lo.y, lo.z, lo.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const uint32_t off = tile + sw128(d4 * 4 + e, lane * 4);
          *reinterpret_cast<uint32_t*>(sm + SM_VHI + off) = hv[e];
          *reinterpret_cast<uint32_t*>(sm + SM_VLO + off) = lv[e];
        }
      }
  };
  // The staging of K and V hides behind the tensor cores: V of a step is staged while its S = Q K^T runs (the V tile
  // was last read by the previous step's P V, which has been waited for), K of the next step while P V runs (the K
  // tile was last read by this step's Q K^T).
  stage_k(0);
  for (int j = 0; j < steps && alive; j++) {
    const int key0 = j * KB;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor cores read what the threads wrote
    fence_before();
    __syncthreads();                               // tiles complete
    if (tid == 0) {
      fence_after();
      // Q_hi [K_hi | K_lo]^T in one instruction of N = 128 (columns 0..63: hi hi, 64..127: hi lo, added when the scores
      // are read), Q_lo K_hi^T on top of the first 64 columns: 16 instructions per step instead of 24
      constexpr uint32_t idesc2 = idesc_tf32(QB, 2 * KB), idesc1 = idesc_tf32(QB, KB);
      uint32_t acc = 0;
#pragma unroll
      for (int kb = 0; kb < 2; kb++) {
        const uint64_t qh = smem_desc(sm_base + SM_QHI + kb * (QB * 128));
        const uint64_t kk = smem_desc(sm_base + SM_K + kb * (2 * KB * 128));   // rows 0..63 of it are K_hi
#pragma unroll
        for (int s = 0; s < 4; s++) {              // 8 tf32 = 32 bytes along K per instruction: the start address moves by 32 B
          mma_ss(tmem + TM_S, qh + 2 * s, kk + 2 * s, idesc2, acc);
          acc = 1;
          mma_ts(tmem + TM_S, tmem + TM_QLO + kb * 32 + s * 8, kk + 2 * s, idesc1, 1);
        }
      }
      mma_commit(bar_addr);
    }
    stage_v(key0);
    alive = wait_mma();
    if (!alive) break;
    fence_after();

    // the next step's K and V rows on their way into L1 while this step's softmax runs: 2 x 128 lines of 128 bytes, one per thread
    if (j + 1 < steps) {
      const int r = (tid & 127) >> 1, key = key0 + KB + r;
      if (key < p.S) {
        const float* line = (tid < 128 ? kg + (int64_t)key * p.ld_k : vg + (int64_t)key * p.ld_v) + (tid & 1) * 32;
        asm volatile("prefetch.global.L1 [%0];" ::"l"(line));
      }
    }
    // ---- this thread's half row of scores: scale, mask, online softmax, P back to tensor memory
    float s[HALF];
    {
      float s2[HALF];
      ld32(lane_addr + TM_S + half * HALF, s);
      ld32(lane_addr + TM_S2 + half * HALF, s2);
#pragma unroll
      for (int i = 0; i < HALF; i++) s[i] += s2[i];
    }
    const bool edge = (p.causal && key0 + KB - 1 > q0) || key0 + KB > p.S;   // uniform: some entry of this step may be masked
    float mx = __int_as_float(0xff800000);
#pragma unroll
    for (int i = 0; i < HALF; i++) {
      float x = s[i] * p.scale_log2e;
      if (edge) {
        const int kj = key0 + half * HALF + i;
        if (kj >= p.S || (p.causal && kj > qi)) x = __int_as_float(0xff800000);
      }
      s[i] = x;
      mx = fmaxf(mx, x);
    }
    // the other half of the row: warps w and w + 4 meet at a barrier of their own (two barriers follow before the slot
    // is written again)
    row_xchg[half][row] = mx;
    pair_barrier(warp & 3);
    mx = fmaxf(mx, row_xchg[half ^ 1][row]);
    const float m_new = fmaxf(m_run, mx);
    const float m_use = (m_new == __int_as_float(0xff800000)) ? 0.0f : m_new;   // a row with nothing visible yet: p = 0 throughout
    const float alpha = ex2(m_run - m_use);        // 0 on the first step (m_run = -inf)
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < HALF / 16; c++) {
      uint32_t hi[16], lo[16];
#pragma unroll
      for (int i = 0; i < 16; i++) {
        const float pv = ex2(s[c * 16 + i] - m_use);
        sum += pv;
        hi[i] = tf32_rna(pv);
        lo[i] = __float_as_uint(__fsub_rn(pv, __uint_as_float(hi[i])));
      }
      st16(lane_addr + TM_PHI + half * HALF + c * 16, hi);
      st16(lane_addr + TM_PLO + half * HALF + c * 16, lo);
    }
    l_run = l_run * alpha + sum;
    m_run = m_new;
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the V tile written above
    fence_before();
    __syncthreads();
    if (tid == 0) {
      fence_after();
      constexpr uint32_t idesc = idesc_tf32(QB, DH);
      uint32_t acc = 0;
#pragma unroll
      for (int ks = 0; ks < KB / 8; ks++) {        // 8 keys per instruction
        const int kb = ks >> 2, sidx = ks & 3;
        const uint64_t vh = smem_desc(sm_base + SM_VHI + kb * (KB * 128)) + 2 * sidx, vl = smem_desc(sm_base + SM_VLO + kb * (KB * 128)) + 2 * sidx;
        mma_ts(tmem + TM_O, tmem + TM_PLO + ks * 8, vh, idesc, acc);
        acc = 1;
        mma_ts(tmem + TM_O, tmem + TM_PHI + ks * 8, vl, idesc, 1);
        mma_ts(tmem + TM_O, tmem + TM_PHI + ks * 8, vh, idesc, 1);
      }
      mma_commit(bar_addr);
    }
    if (j + 1 < steps) stage_k(key0 + KB);
    alive = wait_mma();
    if (!alive) break;
    fence_after();
    {
      float t[HALF];
      ld32(lane_addr + TM_O + half * HALF, t);
#pragma unroll
      for (int i = 0; i < HALF; i++) o[i] = o[i] * alpha + t[i];
    }
    fence_before();                                // the next step's MMAs overwrite S and O only after these loads
  }

  if (alive) {
    // the row's sum: this thread's half plus the partner's (the last barrier of the loop lies between the last read of
    // the slots and this write)
    row_xchg[half][row] = l_run;
    pair_barrier(warp & 3);
    const float l_row = half == 0 ? l_run + row_xchg[1][row] : row_xchg[0][row] + l_run;   // lower half first, in both threads
    if (qi < p.S) {
      const float inv = 1.0f / l_row;
      float4* dst = reinterpret_cast<float4*>(p.out + ((int64_t)b * p.S + qi) * p.ld_o + (int64_t)h * DH + half * HALF);
#pragma unroll
      for (int d = 0; d < HALF; d += 4) dst[d >> 2] = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
    }
  } else {
    if (tid == 0) atomicOr(p.status, STATUS_SDPA_WAIT_TIMEOUT);
    const uint64_t t0 = gtimer();
    while (gtimer() - t0 < 2000000ull) __nanosleep(1000);      // MMAs still in flight finish before tensor memory is released
  }
  fence_before();
  __syncthreads();
  if (warp == 0) {
    fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TM_COLS) : "memory");
  }
}

}  // namespace

bool sdpa_umma_supported(const float* q, const float* k, const float* v, const float* out, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                         int64_t ld_o, int64_t B, int64_t H, int64_t S, int64_t Dh) {
  auto a16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const int64_t q_blocks = (S + QB - 1) / QB;
  return Dh == DH && a16(q) && a16(k) && a16(v) && a16(out) && ld_q % 4 == 0 && ld_k % 4 == 0 && ld_v % 4 == 0 && ld_o % 4 == 0 &&
         S < (1 << 24) && B * H * q_blocks < (1ll << 31);
}

int launch_sdpa_umma(b200q_ctx* ctx, const float* q, const float* k, const float* v, int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t B,
                     int64_t H, int64_t S, float scale, int causal, float* out, int64_t ld_o) {
  if (!ctx->sdpa_umma_ready) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(sdpa_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SDPA_SMEM));
    ctx->sdpa_umma_ready = true;
  }
  SdpaParams p;
  p.q = q; p.k = k; p.v = v; p.out = out;
  p.ld_q = ld_q; p.ld_k = ld_k; p.ld_v = ld_v; p.ld_o = ld_o;
  p.H = (int)H; p.S = (int)S; p.q_blocks = (int)((S + QB - 1) / QB);
  p.scale_log2e = scale * 1.4426950408889634f;
  p.causal = causal;
  p.status = ctx->status_dev;
  p.limit_ns = (unsigned long long)(ctx->wait_limit_s * 1e9);
  const unsigned grid = (unsigned)(B * H * p.q_blocks);
  sdpa_umma_kernel<<<grid, THREADS, SDPA_SMEM, ctx->stream>>>(p);
  return 0;
}

}  // namespace b200q
