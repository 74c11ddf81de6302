// Quantize / dequantize kernels: HBM-streaming, 128-bit loads and stores where
// the layout allows, warp-shuffle reductions for the per-token range.
//
// What they compute (reference, paths inside the reference project):
//   per token   src/compiler/ir/graph/quantization_types.ts:299-317 (range per row),
//               :266-281 (scale = absMax/127 || 1e-10), :118-130 (codes), :132-141 (dequantize)
//   static      src/compiler/passes/lowering/quant_math.ts:16-34 as emitted by
//               src/backend/cpu/codegen.ts:474-545
//   weights     src/compiler/passes/quantization/quantization_pass.ts:390-400
#include "common.cuh"
#include "kernels.cuh"
#include "quant_math.cuh"

namespace b200q {

namespace {

__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }

// Scale of one row from its NaN-ignoring min and max (quantization_types.ts:308-316, 271-275).
__device__ __forceinline__ double row_scale(float mn_f, float mx_f) {
  double mn = (double)mn_f, mx = (double)mx_f;
  if (!isfinite(mn)) mn = -1.0;
  if (!isfinite(mx)) mx = 1.0;
  if (mn == mx) { mn -= 0.5; mx += 0.5; }
  double absmax = fmax(fabs(mn), fabs(mx));
  double s = absmax / 127.0;
  return (s == 0.0 || s != s) ? 1e-10 : s;
}


// Four codes from one float4 on the fast path (valid while the guard stays safe).
__device__ __forceinline__ uint32_t pack4_fast(const float4& v, float inv, QuantGuard& g) {
  const int c0 = quantize_fast(v.x, inv, g);
  const int c1 = quantize_fast(v.y, inv, g);
  const int c2 = quantize_fast(v.z, inv, g);
  const int c3 = quantize_fast(v.w, inv, g);
  return pack_codes(c0, c1, c2, c3);
}
__device__ __forceinline__ uint32_t pack4_exact_p(const float4& v, double s, float qmin, float qmax) {
  return pack_codes(quantize_exact_p(v.x, s, qmin, qmax), quantize_exact_p(v.y, s, qmin, qmax),
                    quantize_exact_p(v.z, s, qmin, qmax), quantize_exact_p(v.w, s, qmin, qmax));
}
__device__ __forceinline__ uint32_t pack4_exact_c(const float4& v, double s, float zp, float qmin, float qmax) {
  return pack_codes(quantize_exact_c(v.x, s, zp, qmin, qmax), quantize_exact_c(v.y, s, zp, qmin, qmax),
                    quantize_exact_c(v.z, s, zp, qmin, qmax), quantize_exact_c(v.w, s, zp, qmin, qmax));
}
__device__ __forceinline__ float guard_limit(float qmin, float qmax) { return fminf(-qmin, qmax) + 0.49f; }

__device__ __forceinline__ bool is_normal_f32(float v) {
  float a = fabsf(v);
  return a >= 1.17549435e-38f && a <= 3.402823466e38f;
}

// ---------------------------------------------------------------------------
// Per-token quantize, row resident in registers.
// A group of G threads owns one row of K = 4*K4 floats; each thread holds VPT
// float4 vectors (coalesced: vector i of a thread is G vectors after vector i-1).
// One read of x, one write of q: 5 bytes per element of HBM traffic.
// Blocks are persistent and software pipelined: the loads of a thread's next row
// are issued before the current row is reduced and encoded, so a block keeps a
// whole row of reads in flight through every phase of its work.
// ---------------------------------------------------------------------------
template <int VPT>
__device__ __forceinline__ void load_row(float4 (&v)[VPT], const float* __restrict__ x, int64_t row, int64_t M, int K4, int G, int t) {
  const float qnan = __int_as_float(0x7fc00000);  // neutral for fminf / fmaxf
  const float4* xr = reinterpret_cast<const float4*>(x) + row * K4;
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    const int c = t + i * G;
    v[i] = (row < M && c < K4) ? ld_stream(xr + c) : make_float4(qnan, qnan, qnan, qnan);
  }
}

// MAXT: largest block the instance is launched with (256 or 1024); the 1024-thread instances have only 64
// registers per thread and do not prefetch.
template <int VPT, int MAXT>
__global__ void __launch_bounds__(MAXT) quantize_per_token_vec_kernel(const float* __restrict__ x, int64_t M, int K4, int G,
                                                                       int8_t* __restrict__ q, float* __restrict__ scales,
                                                                       float qmin, float qmax) {
  __shared__ float s_mn[2][32], s_mx[2][32];
  const int rows_per_block = blockDim.x / G;
  const int grp = threadIdx.x / G;
  const int t = threadIdx.x - grp * G;
  const int64_t row_stride = (int64_t)gridDim.x * rows_per_block;
  const float limit = guard_limit(qmin, qmax);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMM that follows may start its set-up early
  constexpr bool PREFETCH = MAXT <= 256;
  float4 nxt[PREFETCH ? VPT : 1];
  if (PREFETCH) load_row<VPT>(reinterpret_cast<float4(&)[VPT]>(nxt), x, (int64_t)blockIdx.x * rows_per_block + grp, M, K4, G, t);

  int it = 0;
  for (int64_t row0 = (int64_t)blockIdx.x * rows_per_block; row0 < M; row0 += row_stride, it++) {  // row0: uniform per block
    const int64_t row = row0 + grp;
    const bool live = row < M;
    float4 v[VPT];
    if (PREFETCH) {
#pragma unroll
      for (int i = 0; i < VPT; i++) v[i] = nxt[PREFETCH ? i : 0];
      load_row<VPT>(reinterpret_cast<float4(&)[VPT]>(nxt), x, row + row_stride, M, K4, G, t);
    } else {
      load_row<VPT>(v, x, row, M, K4, G, t);
    }

    float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
#pragma unroll
    for (int i = 0; i < VPT; i++) {  // fminf/fmaxf drop NaN operands, as the strict < and > of the reference do
      mn = fminf(fminf(mn, v[i].x), fminf(fminf(v[i].y, v[i].z), v[i].w));
      mx = fmaxf(fmaxf(mx, v[i].x), fmaxf(fmaxf(v[i].y, v[i].z), v[i].w));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (G > 32) {
      // Two buffers alternate, so one barrier per row is enough: a buffer is rewritten two rows later,
      // after every thread has passed the barrier of the row in between.
      const int warp = threadIdx.x >> 5, b = it & 1;
      if ((threadIdx.x & 31) == 0) { s_mn[b][warp] = mn; s_mx[b][warp] = mx; }
      __syncthreads();
      const int w0 = (grp * G) >> 5, nw = G >> 5;
      float lo = s_mn[b][w0], hi = s_mx[b][w0];
      for (int w = 1; w < nw; w++) { lo = fminf(lo, s_mn[b][w0 + w]); hi = fmaxf(hi, s_mx[b][w0 + w]); }
      mn = lo; mx = hi;
    }
    if (!live) continue;

    // Ordinary row (finite, not constant): the reciprocal scale 127/absmax is needed in binary32 only.
    // Everything else (a constant row, whose range is widened in binary64; non-finite ends; a reciprocal
    // that is not a normal binary32 number) encodes through the exact binary64 path.
    const float absmax = fmaxf(fabsf(mn), fabsf(mx));
    const float inv = __fdiv_rn(127.0f, absmax);
    const bool exact_only = !((mn < mx) && absmax <= 3.402823466e38f && is_normal_f32(inv));
#pragma unroll
    for (int i = 0; i < VPT; i++)
      if (t + i * G >= K4) v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);  // dead vectors must not trip the guard

    uint32_t words[VPT];
    QuantGuard guard;
#pragma unroll
    for (int i = 0; i < VPT; i++) words[i] = pack4_fast(v[i], inv, guard);
    if (exact_only || guard.unsafe(limit)) {  // rare: a tie, an out-of-range or a non-finite element
      const double s = row_scale(mn, mx);
#pragma unroll
      for (int i = 0; i < VPT; i++) words[i] = pack4_exact_p(v[i], s, qmin, qmax);
    }
    uint32_t* qr = reinterpret_cast<uint32_t*>(q) + row * K4;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int c = t + i * G;
      if (c < K4) __stcs(qr + c, words[i]);
    }
    // fround(absmax / 127) of two binary32 numbers is the correctly rounded binary32 quotient
    // (rounding the binary64 quotient again is innocuous for a division), so ordinary rows need no binary64.
    if (t == 0) scales[row] = exact_only ? (float)row_scale(mn, mx) : __fdiv_rn(absmax, 127.0f);
  }
}

// ---------------------------------------------------------------------------
// Per-token quantize, rows staged in shared memory by bulk copies.
//
// One persistent block per SM.  A producer lane streams row chunks (R consecutive rows = one contiguous
// range of global memory) into a ring of shared-memory slots with cp.async.bulk; the copy engine keeps the
// whole ring (~190 KB per SM) in flight whatever the warps are doing, which is what saturates HBM.  Each of the
// 16 consumer warps takes every 16th chunk: it reads a row twice from shared memory (min/max, then encode), so
// global memory is read exactly once, reductions never leave the warp (shuffles only, no block barrier), and the
// codes go out as coalesced 128-byte stores.
// A slot is consumed by different warps on successive turns, and a parity wait must never look at a barrier that is
// a whole phase behind (it would pass at once).  Each slot therefore carries a turn counter: the warp that takes
// turn t of a slot first waits until the warp of turn t-1 has released it, and only then waits for the copy.
// Waits are bounded like those of the GEMM: a wait that runs out sets STATUS_QUANT_WAIT_TIMEOUT and the block leaves.
// ---------------------------------------------------------------------------
constexpr int QT_CONSUMER_WARPS = 16;
constexpr int QT_THREADS = 32 * (QT_CONSUMER_WARPS + 1);
constexpr int QT_MAX_SLOTS = 24;

__device__ __forceinline__ uint32_t q_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool q_mbar_try_wait(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ bool q_mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, unsigned long long limit_ns) {
  if (q_mbar_try_wait(bar, parity)) return true;
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  uint32_t it = 0;
  while (!q_mbar_try_wait(bar, parity)) {
    if ((++it & 31u) == 0u) {
      if (*abort_flag) return false;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > limit_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

// Three-input min / max that PROPAGATE NaN (one instruction on sm_100).
__device__ __forceinline__ float fmin3n(float a, float b, float c) {
  float r;
  asm("min.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float fmax3n(float a, float b, float c) {
  float r;
  asm("max.NaN.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// NW consumer warps.  VPT == 0: rows of any length, both passes read the slot.  VPT > 0: one row per slot, K4 == 32 * VPT
// (VPT a multiple of 4): the warp moves its row into registers (VPT float4 per lane), hands the slot back at once and
// does both passes from registers -- a slot is then busy for the time of the copy instead of the time of the encode,
// and the ring no longer runs out of free slots while loads are in flight (NW shrinks as VPT grows: register file).
template <int NW, int VPT>
__global__ void __launch_bounds__(32 * (NW + 1), 1)
quantize_per_token_staged_kernel(const float* __restrict__ x, int64_t M, int K4, int rows_per_chunk, int slots,
                                 int8_t* __restrict__ q, float* __restrict__ scales, float qmin, float qmax, uint32_t* status,
                                 unsigned long long limit_ns) {
  extern __shared__ __align__(128) uint8_t qt_smem[];
  __shared__ uint64_t full[QT_MAX_SLOTS], empty[QT_MAX_SLOTS];
  __shared__ int turn_done[QT_MAX_SLOTS];   // turns of each slot that have been consumed and released
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  volatile int* turns = turn_done;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_bytes = (int64_t)K4 * 16;
  const int64_t chunk_bytes = row_bytes * rows_per_chunk;
  const int64_t num_chunks = (M + rows_per_chunk - 1) / rows_per_chunk;
  // A kernel launched as this one's programmatic dependent (the GEMM of b200q_linear_f32) may take over each SM as
  // soon as this block leaves it and do its set-up there; it waits for this whole grid before it reads anything.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // ... and this kernel may itself have been launched while its predecessor on the stream (which may have produced x)
  // was still draining: nothing is read before that kernel has completed.  A no-op for an ordinary launch.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int s = 0; s < slots; s++) {
      turn_done[s] = 0;
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(q_smem_u32(&full[s])), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(q_smem_u32(&empty[s])), "r"(1) : "memory");
    }
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == NW) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t i = 0;
      for (int64_t chunk = blockIdx.x; chunk < num_chunks; chunk += gridDim.x, i++) {
        const int s = i % slots;
        const uint32_t ph = (i / slots) & 1u;
        if (!q_mbar_wait(q_smem_u32(&empty[s]), ph ^ 1u, abort_flag, limit_ns)) {
          atomicOr(status, STATUS_QUANT_WAIT_TIMEOUT);
          break;
        }
        const int64_t row0 = chunk * rows_per_chunk;
        const int64_t rows = (M - row0 < rows_per_chunk) ? (M - row0) : rows_per_chunk;
        const uint32_t bytes = (uint32_t)(rows * row_bytes);
        const uint32_t bar = q_smem_u32(&full[s]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         q_smem_u32(qt_smem + (int64_t)s * chunk_bytes)),
                     "l"(reinterpret_cast<const uint8_t*>(x) + row0 * row_bytes), "r"(bytes), "r"(bar)
                     : "memory");
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    const float limit = guard_limit(qmin, qmax);
    uint32_t i = 0;
    for (int64_t chunk = blockIdx.x; chunk < num_chunks; chunk += gridDim.x, i++) {
      if ((int)(i % NW) != warp) continue;   // uniform per warp
      const int s = i % slots;
      const int turn = (int)(i / slots);
      const uint32_t ph = (uint32_t)turn & 1u;
      bool ok = true;
      if (lane == 0) {
        // wait for the previous turn of this slot to be released (bounded), then for this turn's copy
        unsigned long long t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        uint32_t spins = 0;
        while (turns[s] != turn) {
          __nanosleep(32);
          if ((++spins & 31u) == 0u) {
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (*abort_flag || t1 - t0 > limit_ns) { *abort_flag = 1; ok = false; break; }
          }
        }
        ok = ok && q_mbar_wait(q_smem_u32(&full[s]), ph, abort_flag, limit_ns);
        if (!ok) atomicOr(status, STATUS_QUANT_WAIT_TIMEOUT);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      const int64_t row0 = chunk * rows_per_chunk;
      const int rows = (int)((M - row0 < rows_per_chunk) ? (M - row0) : rows_per_chunk);
      const float4* slot = reinterpret_cast<const float4*>(qt_smem + (int64_t)s * chunk_bytes);
      if (VPT > 0) {
        constexpr int V = VPT > 0 ? VPT : 4;
        float4 v[V];
#pragma unroll
        for (int j = 0; j < V; j++) v[j] = slot[lane + 32 * j];
        // the row is in registers: hand the slot back before any arithmetic
        __syncwarp();
        if (lane == 0) {
          turns[s] = turn + 1;
          __threadfence_block();
          asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(q_smem_u32(&empty[s])) : "memory");
        }
        float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
        float mn2 = mn, mx2 = mx;
#pragma unroll
        for (int j = 0; j < V; j += 2) {   // NaN-propagating, two chains per bound (see the two-pass form below)
          mn = fmin3n(mn, v[j].x, v[j].y); mx = fmax3n(mx, v[j].x, v[j].y);
          mn2 = fmin3n(mn2, v[j].z, v[j].w); mx2 = fmax3n(mx2, v[j].z, v[j].w);
          mn = fmin3n(mn, v[j + 1].x, v[j + 1].y); mx = fmax3n(mx, v[j + 1].x, v[j + 1].y);
          mn2 = fmin3n(mn2, v[j + 1].z, v[j + 1].w); mx2 = fmax3n(mx2, v[j + 1].z, v[j + 1].w);
        }
        mn = fmin3n(mn, mn, mn2); mx = fmax3n(mx, mx, mx2);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          mn = fmin3n(mn, mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mx = fmax3n(mx, mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const bool nan_row = (mn != mn) || (mx != mx);
        if (nan_row) {   // the reference's strict comparisons ignore NaN: rescan with the NaN-dropping forms
          mn = __int_as_float(0x7f800000); mx = __int_as_float(0xff800000);
#pragma unroll
          for (int j = 0; j < V; j++) {
            mn = fminf(fminf(mn, v[j].x), fminf(fminf(v[j].y, v[j].z), v[j].w));
            mx = fmaxf(fmaxf(mx, v[j].x), fmaxf(fmaxf(v[j].y, v[j].z), v[j].w));
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          }
        }
        const float absmax = fmaxf(fabsf(mn), fabsf(mx));
        const float inv = __fdiv_rn(127.0f, absmax);
        const bool exact_only = nan_row || limit < 127.0f || !((mn < mx) && absmax <= 3.402823466e38f && is_normal_f32(inv));
        uint32_t* qr = reinterpret_cast<uint32_t*>(q) + row0 * K4 + lane;
        // The unrolled body holds the fast encode only.  Groups that come near a tie are noted and redone afterwards,
        // and odd rows are encoded entirely, from the row in global memory (just read, so in L2): rare, and it keeps
        // the register copy of the row statically indexed and the binary64 code out of the unrolled loop.
        const float4* xg = reinterpret_cast<const float4*>(x) + row0 * K4 + lane;
        uint32_t redo = 0;
        if (!exact_only) {
          const uint64_t inv2 = f2_pack(inv, inv), magic2 = f2_pack(12582912.0f, 12582912.0f);
#pragma unroll
          for (int g = 0; g < V; g += 4) {
            float far = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) __stcs(qr + 32 * (g + j), pack4_fast_lean(v[g + j], inv2, magic2, far));
            redo |= (far >= 0.49993920f) ? (1u << (g / 4)) : 0u;       // 0.5 - 127.5 * 2^-21
          }
        } else {
          redo = (V / 4 >= 32) ? 0xffffffffu : ((1u << (V / 4)) - 1u);
        }
        while (redo) {
          const int g = (__ffs((int)redo) - 1) * 4;
          redo &= redo - 1;
          float4 t[4];
          int tie = 0;
#pragma unroll
          for (int j = 0; j < 4; j++) {
            t[j] = xg[32 * (g + j)];
            (void)quantize_fast_bounded(t[j].x, inv, tie); (void)quantize_fast_bounded(t[j].y, inv, tie);
            (void)quantize_fast_bounded(t[j].z, inv, tie); (void)quantize_fast_bounded(t[j].w, inv, tie);
          }
          if (exact_only || tie >= 0x3f000000) {
            const double sd = row_scale(mn, mx);
#pragma unroll
            for (int j = 0; j < 4; j++) __stcs(qr + 32 * (g + j), pack4_exact_p(t[j], sd, qmin, qmax));
          }
        }
        if (lane == 0) scales[row0] = exact_only ? (float)row_scale(mn, mx) : __fdiv_rn(absmax, 127.0f);
        continue;
      }
      for (int r = 0; r < rows; r++) {
        const float4* xr = slot + (int64_t)r * K4;
        // pass 1: range of the row with NaN-PROPAGATING three-input min / max (one instruction per two elements and
        // bound).  A row that contains a NaN shows up as a NaN range: it is rescanned with the NaN-dropping forms
        // (the reference's strict comparisons ignore NaN) and encoded entirely on the exact path.
        float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
        int c = lane;
#pragma unroll 2
        for (; c + 96 < K4; c += 128) {
          const float4 v0 = xr[c], v1 = xr[c + 32], v2 = xr[c + 64], v3 = xr[c + 96];
          float mn2 = fmin3n(v0.x, v0.y, v0.z), mx2 = fmax3n(v0.x, v0.y, v0.z);   // two independent chains per bound
          mn = fmin3n(mn, v0.w, v1.x); mx = fmax3n(mx, v0.w, v1.x);
          mn2 = fmin3n(mn2, v1.y, v1.z); mx2 = fmax3n(mx2, v1.y, v1.z);
          mn = fmin3n(mn, v1.w, v2.x); mx = fmax3n(mx, v1.w, v2.x);
          mn2 = fmin3n(mn2, v2.y, v2.z); mx2 = fmax3n(mx2, v2.y, v2.z);
          mn = fmin3n(mn, v2.w, v3.x); mx = fmax3n(mx, v2.w, v3.x);
          mn2 = fmin3n(mn2, v3.y, v3.z); mx2 = fmax3n(mx2, v3.y, v3.z);
          mn = fmin3n(mn, v3.w, mn2); mx = fmax3n(mx, v3.w, mx2);
        }
        for (; c < K4; c += 32) {
          const float4 v = xr[c];
          mn = fmin3n(fmin3n(mn, v.x, v.y), v.z, v.w);
          mx = fmax3n(fmax3n(mx, v.x, v.y), v.z, v.w);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          mn = fmin3n(mn, mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mx = fmax3n(mx, mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        const bool nan_row = (mn != mn) || (mx != mx);   // uniform over the warp after the reduction
        if (nan_row) {
          mn = __int_as_float(0x7f800000); mx = __int_as_float(0xff800000);
          for (int cc = lane; cc < K4; cc += 32) {
            const float4 v = xr[cc];
            mn = fminf(fminf(mn, v.x), fminf(fminf(v.y, v.z), v.w));
            mx = fmaxf(fmaxf(mx, v.x), fmaxf(fmaxf(v.y, v.z), v.w));
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
          }
        }
        const float absmax = fmaxf(fabsf(mn), fabsf(mx));
        const float inv = __fdiv_rn(127.0f, absmax);
        // odd rows (constant, non-finite ends, NaN inside, a reciprocal that is not a normal number) and narrow clamps
        // encode through binary64 throughout
        const bool exact_only = nan_row || limit < 127.0f || !((mn < mx) && absmax <= 3.402823466e38f && is_normal_f32(inv));
        uint32_t* qr = reinterpret_cast<uint32_t*>(q) + (row0 + r) * K4;
        if (!exact_only && (K4 & 127) == 0) {
          // pass 2, ordinary row whose length is a multiple of 512 elements: no bounds checks, five instructions per
          // element for the code, one more to keep the largest |t - rint t| of the 16 elements a lane handles per turn.
          // Every element is finite here and |t| <= 127 (1 + 2^-23), so a tie is the only thing that can go wrong:
          // first a cheap test with the worst-case margin (|t| = 127.5), and only if that trips the per-element one.
          const uint64_t inv2 = f2_pack(inv, inv), magic2 = f2_pack(12582912.0f, 12582912.0f);
          for (int c0 = lane; c0 < K4; c0 += 128) {
            float4 v[4];
            uint32_t w[4];
            float far = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) v[j] = xr[c0 + 32 * j];
#pragma unroll
            for (int j = 0; j < 4; j++) w[j] = pack4_fast_lean(v[j], inv2, magic2, far);
            if (far >= 0.49993920f) {                                   // 0.5 - 127.5 * 2^-21
              int tie = 0;
#pragma unroll
              for (int j = 0; j < 4; j++) {
                (void)quantize_fast_bounded(v[j].x, inv, tie); (void)quantize_fast_bounded(v[j].y, inv, tie);
                (void)quantize_fast_bounded(v[j].z, inv, tie); (void)quantize_fast_bounded(v[j].w, inv, tie);
              }
              if (tie >= 0x3f000000) {
                const double sd = row_scale(mn, mx);
#pragma unroll
                for (int j = 0; j < 4; j++) w[j] = pack4_exact_p(v[j], sd, qmin, qmax);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; j++) __stcs(qr + c0 + 32 * j, w[j]);
          }
        } else {
          // pass 2, general: ragged row length or the exact path
          for (int c0 = lane; c0 < K4; c0 += 128) {
            float4 v[4];
            uint32_t w[4];
            int tie = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int cc = c0 + 32 * j;
              v[j] = (cc < K4) ? xr[cc] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int j = 0; j < 4; j++)
              w[j] = pack_codes(quantize_fast_bounded(v[j].x, inv, tie), quantize_fast_bounded(v[j].y, inv, tie),
                                quantize_fast_bounded(v[j].z, inv, tie), quantize_fast_bounded(v[j].w, inv, tie));
            if (exact_only || tie >= 0x3f000000) {  // rare: a tie, NaN, an odd row, a narrow clamp
              const double sd = row_scale(mn, mx);
#pragma unroll
              for (int j = 0; j < 4; j++) w[j] = pack4_exact_p(v[j], sd, qmin, qmax);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int cc = c0 + 32 * j;
              if (cc < K4) __stcs(qr + cc, w[j]);
            }
          }
        }
        if (lane == 0) scales[row0 + r] = exact_only ? (float)row_scale(mn, mx) : __fdiv_rn(absmax, 127.0f);
      }
      // every lane has finished reading the slot: hand it back to the producer
      __syncwarp();
      if (lane == 0) {
        turns[s] = turn + 1;
        __threadfence_block();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(q_smem_u32(&empty[s])) : "memory");
      }
    }
  }
  if (*abort_flag) {  // give copies in flight time to land before the shared memory is released (bounded: 2 ms)
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    do {
      __nanosleep(1000);
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    } while (t1 - t0 < 2000000ull);
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------
// Per-token quantize, a team of TEAM warps per row, the row in registers straight from global memory.
// Warp p of a team holds vectors [p * 32 * VPT, (p + 1) * 32 * VPT) of the row; lane l loads float4 number
// l + 32 j of that part (j < VPT): every load instruction of a warp covers 512 contiguous bytes, all VPT of them are
// issued before the first use.  TEAM == 1: nothing but the warp itself is involved afterwards (shuffle reductions, no
// shared memory, no barrier, no producer).  TEAM > 1: the warps of a team exchange their partial range through
// shared memory and a named barrier of their own, once per row.  Parts shorter than 32 * VPT vectors repeat the
// row's first vectors in the unused registers (harmless to the range, never stored).  Short rows leave room for many
// warps per SM, whose loads overlap each other's arithmetic; long rows are split so that a warp keeps few enough
// registers for that to stay true.
// ---------------------------------------------------------------------------
// Named barrier of one team (a block holds at most two teams of more than one warp).  The barrier number is an
// immediate, so that the kernel reserves the barriers it uses and no more (a register operand reserves all sixteen,
// which limits the blocks per SM).
template <int TEAM>
__device__ __forceinline__ void team_barrier(int team) {
  if (team == 0) asm volatile("bar.sync 1, %0;" ::"n"(32 * TEAM) : "memory");
  else asm volatile("bar.sync 2, %0;" ::"n"(32 * TEAM) : "memory");
}

template <int TEAM>
__device__ __forceinline__ void team_exchange(float& mn, float& mx, float2* slots, int team, int part, int lane, bool nan_dropping) {
  if (TEAM == 1) return;
  if (lane == 0) slots[team * TEAM + part] = make_float2(mn, mx);
  team_barrier<TEAM>(team);
#pragma unroll
  for (int p = 0; p < TEAM; p++) {
    const float2 o = slots[team * TEAM + p];
    if (nan_dropping) { mn = fminf(mn, o.x); mx = fmaxf(mx, o.y); }
    else { mn = fmin3n(mn, mn, o.x); mx = fmax3n(mx, mx, o.y); }
  }
  team_barrier<TEAM>(team);   // the slots may be written again
}

// KEYS: the rows' ranges are given (order-preserving keys published by the kernel that produced x, [0, M) maxima and
// [M, 2M) minima), so the range pass and the exchange fall away and the kernel is one streaming pass; rows may then
// hold NaN or infinite elements the kernel has not looked for, which the encode notices by itself.  ld_in4 / ld_out4:
// row strides of x and q in units of four elements.
template <int VPT, int TEAM, int WARPS, bool KEYS>
__global__ void __launch_bounds__(32 * WARPS) quantize_per_token_warp_kernel(const float* __restrict__ x, int64_t M, int K4,
                                                                             int64_t ld_in4, int64_t ld_out4,
                                                                             const uint32_t* __restrict__ keys,
                                                                             int8_t* __restrict__ q, float* __restrict__ scales,
                                                                             float qmin, float qmax) {
  static_assert(VPT % 4 == 0 && WARPS % TEAM == 0, "the encode works on groups of four vectors; whole teams per block");
  static_assert(TEAM == 1 || WARPS / TEAM <= 2, "team_barrier knows two barriers");
  __shared__ float2 slots[(TEAM > 1 && !KEYS) ? WARPS : 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int team = warp / TEAM, part = warp - team * TEAM;
  const int64_t row = (int64_t)blockIdx.x * (WARPS / TEAM) + team;
  const float limit = guard_limit(qmin, qmax);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMM that follows may start its set-up early
  asm volatile("griddepcontrol.wait;" ::: "memory");                // ... and x may come from the kernel before this one
  if (row >= M) return;                                             // whole teams leave together
  const int c0 = part * 32 * VPT + lane;                            // this lane's first vector of the row
  const float4* xrow = reinterpret_cast<const float4*>(x) + row * ld_in4;
  float4 v[VPT];
#pragma unroll
  for (int j = 0; j < VPT; j++) v[j] = ld_stream(xrow + ((c0 + 32 * j < K4) ? c0 + 32 * j : lane));
  float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
  bool nan_row = false;
  if (KEYS) {
    mx = range_max_from_key(__ldg(keys + row));
    mn = range_min_from_key(__ldg(keys + M + row));
  } else {
    float mn2 = mn, mx2 = mx;
#pragma unroll
    for (int j = 0; j < VPT; j += 2) {   // NaN-propagating three-input forms, two chains per bound
      mn = fmin3n(mn, v[j].x, v[j].y); mx = fmax3n(mx, v[j].x, v[j].y);
      mn2 = fmin3n(mn2, v[j].z, v[j].w); mx2 = fmax3n(mx2, v[j].z, v[j].w);
      mn = fmin3n(mn, v[j + 1].x, v[j + 1].y); mx = fmax3n(mx, v[j + 1].x, v[j + 1].y);
      mn2 = fmin3n(mn2, v[j + 1].z, v[j + 1].w); mx2 = fmax3n(mx2, v[j + 1].z, v[j + 1].w);
    }
    mn = fmin3n(mn, mn, mn2); mx = fmax3n(mx, mx, mx2);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fmin3n(mn, mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmax3n(mx, mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    team_exchange<TEAM>(mn, mx, slots, team, part, lane, false);
    nan_row = (mn != mn) || (mx != mx);                               // the same in every warp of the team
    if (nan_row) {   // the reference's strict comparisons ignore NaN: rescan with the NaN-dropping forms
      mn = __int_as_float(0x7f800000); mx = __int_as_float(0xff800000);
#pragma unroll
      for (int j = 0; j < VPT; j++) {
        mn = fminf(fminf(mn, v[j].x), fminf(fminf(v[j].y, v[j].z), v[j].w));
        mx = fmaxf(fmaxf(mx, v[j].x), fmaxf(fmaxf(v[j].y, v[j].z), v[j].w));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      }
      team_exchange<TEAM>(mn, mx, slots, team, part, lane, true);
    }
  }
  const float absmax = fmaxf(fabsf(mn), fabsf(mx));
  const float inv = __fdiv_rn(127.0f, absmax);
  const bool exact_only = nan_row || limit < 127.0f || !((mn < mx) && absmax <= 3.402823466e38f && is_normal_f32(inv));
  uint32_t* qr = reinterpret_cast<uint32_t*>(q) + row * ld_out4 + c0;
  uint32_t redo = 0;
  if (!exact_only) {
    const uint64_t inv2 = f2_pack(inv, inv), magic2 = f2_pack(12582912.0f, 12582912.0f);
#pragma unroll
    for (int g = 0; g < VPT; g += 4) {
      float far = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const uint32_t w = KEYS ? pack4_fast_lean_nan(v[g + j], inv2, magic2, far) : pack4_fast_lean(v[g + j], inv2, magic2, far);
        if (c0 + 32 * (g + j) < K4) __stcs(qr + 32 * (g + j), w);
      }
      redo |= !(far < 0.49993920f) ? (1u << (g / 4)) : 0u;       // 0.5 - 127.5 * 2^-21; a NaN counts as near
    }
  } else {
    redo = (1u << (VPT / 4)) - 1u;
  }
  // Groups that came near a tie, and odd rows entirely, are redone from global memory (just read, so from L2) with
  // the exact routine: rare, and it keeps the register copy statically indexed and binary64 out of the unrolled body.
  while (redo) {
    const int g = (__ffs((int)redo) - 1) * 4;
    redo &= redo - 1;
    const double sd = row_scale(mn, mx);
    for (int j = 0; j < 4; j++) {
      if (c0 + 32 * (g + j) >= K4) continue;
      const float4 t = xrow[c0 + 32 * (g + j)];
      int tie = 0;
      (void)quantize_fast_bounded(t.x, inv, tie); (void)quantize_fast_bounded(t.y, inv, tie);
      (void)quantize_fast_bounded(t.z, inv, tie); (void)quantize_fast_bounded(t.w, inv, tie);
      if (exact_only || tie >= 0x3f000000) __stcs(qr + 32 * (g + j), pack4_exact_p(t, sd, qmin, qmax));
    }
  }
  if (lane == 0 && part == 0 && scales) scales[row] = exact_only ? (float)row_scale(mn, mx) : __fdiv_rn(absmax, 127.0f);
}

// Any K, any alignment: one block per row, the row is read twice (the second
// read is served by L2 for rows up to tens of megabytes).
__global__ void __launch_bounds__(256) quantize_per_token_generic_kernel(const float* __restrict__ x, int64_t M, int64_t K,
                                                                         int8_t* __restrict__ q, float* __restrict__ scales,
                                                                         float qmin, float qmax) {
  __shared__ float s_mn[8], s_mx[8];
  __shared__ double s_scale;
  __shared__ float s_inv;
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float* xr = x + row * K;
    float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {
      float vv = xr[k];
      mn = fminf(mn, vv);
      mx = fmaxf(mx, vv);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) { s_mn[threadIdx.x >> 5] = mn; s_mx[threadIdx.x >> 5] = mx; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < (int)(blockDim.x >> 5); w++) { mn = fminf(mn, s_mn[w]); mx = fmaxf(mx, s_mx[w]); }
      double s = row_scale(mn, mx);
      s_scale = s;
      s_inv = (float)(1.0 / s);
      scales[row] = (float)s;
    }
    __syncthreads();
    const double s = s_scale;
    const float inv = s_inv;
    const bool exact_only = !is_normal_f32(inv);
    int8_t* qr = q + row * K;
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {
      QuantGuard guard;
      const float xv = xr[k];
      int c = quantize_fast(xv, inv, guard);
      if (exact_only || guard.unsafe(guard_limit(qmin, qmax))) c = quantize_exact_p(xv, s, qmin, qmax);
      qr[k] = (int8_t)c;
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Per-token dequantize: y[m,k] = fround(q[m,k] * scale[m]).  A thread turns VPT
// packed words (4 codes each) into VPT float4 stores.
// ---------------------------------------------------------------------------
template <int VPT>
__global__ void __launch_bounds__(256) dequantize_per_token_vec_kernel(const int8_t* __restrict__ q,
                                                                       const float* __restrict__ scales, int64_t M, int K4,
                                                                       float* __restrict__ y) {
  const int64_t row = blockIdx.x;
  const float s = __ldg(scales + row);
  const uint32_t* qr = reinterpret_cast<const uint32_t*>(q) + row * K4;
  float4* yr = reinterpret_cast<float4*>(y) + row * K4;
  const int base = blockIdx.y * (blockDim.x * VPT) + threadIdx.x;
  uint32_t w[VPT];
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    int c = base + i * blockDim.x;
    w[i] = (c < K4) ? __ldcs(qr + c) : 0u;
  }
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    int c = base + i * blockDim.x;
    if (c < K4) {
      float4 o;
      o.x = __fmul_rn((float)(int8_t)(w[i] & 0xff), s);
      o.y = __fmul_rn((float)(int8_t)((w[i] >> 8) & 0xff), s);
      o.z = __fmul_rn((float)(int8_t)((w[i] >> 16) & 0xff), s);
      o.w = __fmul_rn((float)(int8_t)(w[i] >> 24), s);
      __stcs(yr + c, o);
    }
  }
}

__global__ void __launch_bounds__(256) dequantize_per_token_generic_kernel(const int8_t* __restrict__ q,
                                                                           const float* __restrict__ scales, int64_t M,
                                                                           int64_t K, float* __restrict__ y) {
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float s = scales[row];
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) y[row * K + k] = __fmul_rn((float)q[row * K + k], s);
  }
}

// ---------------------------------------------------------------------------
// Static-scale (compiled-op) quantize / dequantize over a flat tensor.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_static_kernel(const float* __restrict__ x, int64_t n, double s, float inv,
                                                              float zp, int exact_only, float qmin, float qmax,
                                                              int8_t* __restrict__ q, int vec_ok) {
  const bool exact = exact_only != 0;
  // Unsigned targets clamp at 0: the guard (symmetric in |t|) then sends every negative quotient to the exact path.
  const float limit = guard_limit(qmin, qmax);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t n4 = vec_ok ? (n >> 2) : 0;
  const float4* x4 = reinterpret_cast<const float4*>(x);
  uint32_t* q4 = reinterpret_cast<uint32_t*>(q);
  for (int64_t i = tid; i < n4; i += stride) {
    const float4 v = ld_stream(x4 + i);
    QuantGuard guard;
    uint32_t w = pack4_fast(v, inv, guard);
    if (exact || guard.unsafe(limit)) w = pack4_exact_c(v, s, zp, qmin, qmax);
    __stcs(q4 + i, w);
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += stride) {
    QuantGuard guard;
    int c = quantize_fast(x[i], inv, guard);
    if (exact || guard.unsafe(limit)) c = quantize_exact_c(x[i], s, zp, qmin, qmax);
    q[i] = (int8_t)c;
  }
}

// (+q) [fround(- zp)] then fround(* s): the int -> f32 cast is not rounded (cpu/codegen.ts:521).
__device__ __forceinline__ float dequant_c(int qv, double s, float zp) {
  if (zp != 0.0f) return __double2float_rn((double)__double2float_rn((double)qv - (double)zp) * s);
  return __double2float_rn((double)qv * s);
}

// 8-bit sources have 256 possible codes: a shared-memory table of the exact
// results keeps binary64 off the streaming path.  src_kind 0 = i8, 1 = ui8.
__global__ void __launch_bounds__(256) dequantize_static_8_kernel(const uint8_t* __restrict__ q, int64_t n, double s, float zp,
                                                                  int src_kind, float* __restrict__ y, int vec_ok) {
  __shared__ float lut[256];
  {
    int b = threadIdx.x;  // blockDim.x == 256
    int code = src_kind == 0 ? (int)(int8_t)b : b;
    lut[b] = dequant_c(code, s, zp);
  }
  __syncthreads();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t n4 = vec_ok ? (n >> 2) : 0;
  const uint32_t* q4 = reinterpret_cast<const uint32_t*>(q);
  float4* y4 = reinterpret_cast<float4*>(y);
  for (int64_t i = tid; i < n4; i += stride) {
    uint32_t w = __ldcs(q4 + i);
    float4 o = make_float4(lut[w & 0xff], lut[(w >> 8) & 0xff], lut[(w >> 16) & 0xff], lut[w >> 24]);
    __stcs(y4 + i, o);
  }
  for (int64_t i = (n4 << 2) + tid; i < n; i += stride) y[i] = lut[q[i]];
}

__global__ void __launch_bounds__(256) dequantize_static_i32_kernel(const int32_t* __restrict__ q, int64_t n, double s, float zp,
                                                                    float* __restrict__ y) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] = dequant_c(q[i], s, zp);
}

// ---------------------------------------------------------------------------
// Weight preparation (once per model): per-output-channel symmetric scales and
// int8 codes, written K-major ([N,K]) whatever the source layout.
// ---------------------------------------------------------------------------
// layout 0: w is [N,K] (channel = row); layout 1: w is [K,N] (channel = column).
__global__ void __launch_bounds__(256) weight_range_kernel(const float* __restrict__ w, int64_t N, int64_t K, int layout,
                                                           double* __restrict__ scales64, float* __restrict__ scales32) {
  __shared__ float s_mn[8], s_mx[8];
  for (int64_t n = blockIdx.x; n < N; n += gridDim.x) {
    float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
    for (int64_t k = threadIdx.x; k < K; k += blockDim.x) {
      float v = layout == 0 ? w[n * K + k] : w[k * N + n];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) { s_mn[threadIdx.x >> 5] = mn; s_mx[threadIdx.x >> 5] = mx; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int wi = 1; wi < (int)(blockDim.x >> 5); wi++) { mn = fminf(mn, s_mn[wi]); mx = fmaxf(mx, s_mx[wi]); }
      double s = row_scale(mn, mx);
      if (scales64) scales64[n] = s;
      if (scales32) scales32[n] = (float)s;
    }
    __syncthreads();
  }
}

// 32x32 tile through shared memory so that both the read (source layout) and
// the write ([N,K]) are coalesced.  Every code takes the exact binary64 path:
// this runs once per weight.
__global__ void __launch_bounds__(256) weight_quantize_kernel(const float* __restrict__ w, int64_t N, int64_t K, int layout,
                                                              const double* __restrict__ scales64, float qmin, float qmax,
                                                              int8_t* __restrict__ qw) {
  __shared__ float tile[32][33];
  const int64_t n0 = (int64_t)blockIdx.y * 32, k0 = (int64_t)blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int j = ty; j < 32; j += 8) {
    if (layout == 0) {
      int64_t n = n0 + j, k = k0 + tx;
      tile[j][tx] = (n < N && k < K) ? w[n * K + k] : 0.0f;  // tile[n][k]
    } else {
      int64_t k = k0 + j, n = n0 + tx;
      tile[tx][j] = (n < N && k < K) ? w[k * N + n] : 0.0f;  // tile[n][k]
    }
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    int64_t n = n0 + j, k = k0 + tx;
    if (n < N && k < K) qw[n * K + k] = (int8_t)quantize_exact_p(tile[j][tx], scales64[n], qmin, qmax);
  }
}

// int8 [K,N] -> [N,K]
__global__ void __launch_bounds__(256) transpose_i8_kernel(const int8_t* __restrict__ src, int64_t K, int64_t N,
                                                           int8_t* __restrict__ dst) {
  __shared__ int8_t tile[32][33];
  const int64_t n0 = (int64_t)blockIdx.y * 32, k0 = (int64_t)blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8) {
    int64_t k = k0 + j, n = n0 + tx;
    tile[j][tx] = (k < K && n < N) ? src[k * N + n] : (int8_t)0;
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    int64_t n = n0 + j, k = k0 + tx;
    if (n < N && k < K) dst[n * K + k] = tile[tx][j];
  }
}

// ---------------------------------------------------------------------------
// Column-sharded (N-sharded) layers: a row of the activation is spread over several GPUs, so its range is
// found in two steps (range of the local columns here, min / max over the GPUs by the host's collective) and
// the codes are then computed from the agreed range - bit for bit what quantizing the whole row would give.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) row_range_kernel(const float* __restrict__ y, int64_t M, int64_t N, int64_t ld,
                                                        float* __restrict__ mn_out, float* __restrict__ mx_out) {
  __shared__ float s_mn[8], s_mx[8];
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float* yr = y + row * ld;
    float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
    for (int64_t k = threadIdx.x; k < N; k += blockDim.x) {
      const float v = yr[k];
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) { s_mn[threadIdx.x >> 5] = mn; s_mx[threadIdx.x >> 5] = mx; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < (int)(blockDim.x >> 5); w++) { mn = fminf(mn, s_mn[w]); mx = fmaxf(mx, s_mx[w]); }
      mn_out[row] = mn;
      mx_out[row] = mx;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256) quantize_rows_with_range_kernel(const float* __restrict__ y, int64_t M, int64_t N, int64_t ld_in,
                                                                       const float* __restrict__ mn_in, const float* __restrict__ mx_in,
                                                                       int8_t* __restrict__ q, int64_t ld_out, float* __restrict__ scales,
                                                                       float qmin, float qmax) {
  const float limit = guard_limit(qmin, qmax);
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float mn = mn_in[row], mx = mx_in[row];
    const float absmax = fmaxf(fabsf(mn), fabsf(mx));
    const float inv = __fdiv_rn(127.0f, absmax);
    const bool exact_only = !((mn < mx) && absmax <= 3.402823466e38f && is_normal_f32(inv));
    const double s = row_scale(mn, mx);
    const float* yr = y + row * ld_in;
    int8_t* qr = q + row * ld_out;
    for (int64_t k = threadIdx.x; k < N; k += blockDim.x) {
      QuantGuard guard;
      const float xv = yr[k];
      int c = quantize_fast(xv, inv, guard);
      if (exact_only || guard.unsafe(limit)) c = quantize_exact_p(xv, s, qmin, qmax);
      qr[k] = (int8_t)c;
    }
    if (threadIdx.x == 0 && scales) scales[row] = (float)s;
  }
}

// The same second step when the ranges arrive as keys (range_key_max / range_key_min): the kernel that produced y
// published them while the values were in its registers, so this is the only pass over y: 128-bit loads, four codes
// per 32-bit store, four loads in flight per thread.  Needs N % 4 == 0 and 16-byte aligned rows; the generic form
// below it takes everything else.
template <int UNROLL>
__global__ void __launch_bounds__(256) quantize_rows_with_keys_vec_kernel(const float* __restrict__ y, int64_t M, int N4, int64_t ld_in,
                                                                          const uint32_t* __restrict__ keys, int8_t* __restrict__ q,
                                                                          int64_t ld_out, float* __restrict__ scales, float qmin, float qmax) {
  const float limit = guard_limit(qmin, qmax);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMM that follows may start its set-up early
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float mx = range_max_from_key(__ldg(keys + row)), mn = range_min_from_key(__ldg(keys + M + row));
    const float absmax = fmaxf(fabsf(mn), fabsf(mx));
    const float inv = __fdiv_rn(127.0f, absmax);
    const bool exact_only = !((mn < mx) && absmax <= 3.402823466e38f && is_normal_f32(inv));
    const double s = row_scale(mn, mx);
    const float4* yr = reinterpret_cast<const float4*>(y + row * ld_in);
    uint32_t* qr = reinterpret_cast<uint32_t*>(q + row * ld_out);
    for (int k0 = threadIdx.x; k0 < N4; k0 += 256 * UNROLL) {
      float4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; u++) {
        const int k = k0 + u * 256;
        if (k < N4) v[u] = ld_stream(yr + k);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; u++) {
        const int k = k0 + u * 256;
        if (k < N4) {
          QuantGuard guard;
          uint32_t w = pack4_fast(v[u], inv, guard);
          if (exact_only || guard.unsafe(limit)) w = pack4_exact_p(v[u], s, qmin, qmax);
          qr[k] = w;
        }
      }
    }
    if (threadIdx.x == 0 && scales) scales[row] = (float)s;
  }
}

__global__ void __launch_bounds__(256) quantize_rows_with_keys_kernel(const float* __restrict__ y, int64_t M, int64_t N, int64_t ld_in,
                                                                      const uint32_t* __restrict__ keys, int8_t* __restrict__ q,
                                                                      int64_t ld_out, float* __restrict__ scales, float qmin, float qmax) {
  const float limit = guard_limit(qmin, qmax);
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const float mx = range_max_from_key(keys[row]), mn = range_min_from_key(keys[M + row]);
    const float absmax = fmaxf(fabsf(mn), fabsf(mx));
    const float inv = __fdiv_rn(127.0f, absmax);
    const bool exact_only = !((mn < mx) && absmax <= 3.402823466e38f && is_normal_f32(inv));
    const double s = row_scale(mn, mx);
    const float* yr = y + row * ld_in;
    int8_t* qr = q + row * ld_out;
    for (int64_t k = threadIdx.x; k < N; k += blockDim.x) {
      QuantGuard guard;
      const float xv = yr[k];
      int c = quantize_fast(xv, inv, guard);
      if (exact_only || guard.unsafe(limit)) c = quantize_exact_p(xv, s, qmin, qmax);
      qr[k] = (int8_t)c;
    }
    if (threadIdx.x == 0 && scales) scales[row] = (float)s;
  }
}

// Ranges as keys from separate minimum / maximum arrays (the row-range pass), so that column-sharded layers can
// exchange either form with one max-reduction over the GPUs.
__global__ void __launch_bounds__(256) range_to_keys_kernel(const float* __restrict__ mn, const float* __restrict__ mx, int64_t M,
                                                            uint32_t* __restrict__ keys) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M) return;
  const float a = mx[i], b = mn[i];
  keys[i] = (a != a || a == __int_as_float(0xff800000)) ? 0u : range_key_max(a);
  keys[M + i] = (b != b || b == __int_as_float(0x7f800000)) ? 0u : range_key_min(b);
}

// ---------------------------------------------------------------------------
// Calibration observer (min/max mode): running minimum and maximum of every value shown to it, NaN ignored,
// exactly as ValueObserver.update compares (src/compiler/analysis/calibration.ts:24-30).  state[0] = min, state[1] = max.
// Float atomics through the integer ordering of the bit patterns: non-negative floats order like signed integers,
// negative ones like unsigned integers in reverse.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void atomic_max_f32(float* addr, float v) {
  v = __fadd_rn(v, 0.0f);   // -0.0 becomes +0.0: as a bit pattern -0.0 is the smallest integer, not a zero
  if (v >= 0.0f) atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}
__device__ __forceinline__ void atomic_min_f32(float* addr, float v) {
  v = __fadd_rn(v, 0.0f);
  if (v >= 0.0f) atomicMin(reinterpret_cast<int*>(addr), __float_as_int(v));
  else atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

__global__ void __launch_bounds__(256) minmax_observe_kernel(const float* __restrict__ x, int64_t n, float* __restrict__ state) {
  __shared__ float s_mn[8], s_mx[8];
  float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
  const int64_t n4 = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 ? n / 4 : 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x, first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int64_t i = first; i < n4; i += stride) {
    const float4 v = __ldcs(reinterpret_cast<const float4*>(x) + i);
    mn = fminf(fminf(mn, v.x), fminf(fminf(v.y, v.z), v.w));   // fminf / fmaxf drop NaN operands
    mx = fmaxf(fmaxf(mx, v.x), fmaxf(fmaxf(v.y, v.z), v.w));
  }
  for (int64_t i = n4 * 4 + first; i < n; i += stride) {
    mn = fminf(mn, x[i]);
    mx = fmaxf(mx, x[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((threadIdx.x & 31) == 0) { s_mn[threadIdx.x >> 5] = mn; s_mx[threadIdx.x >> 5] = mx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; w++) { mn = fminf(mn, s_mn[w]); mx = fmaxf(mx, s_mx[w]); }
    // +Inf / -Inf are the "nothing seen" values: they leave the state alone
    if (mn != __int_as_float(0x7f800000)) atomic_min_f32(state, mn);
    if (mx != __int_as_float(0xff800000)) atomic_max_f32(state + 1, mx);
  }
}

// Histogram observer (percentile / entropy calibration): HistogramCollector.update's binning
// (src/compiler/analysis/calibration.ts:64-79), idx = min(numBins - 1, floor((v - rangeMin) * (numBins / range))) in
// binary64 as the reference evaluates it; a value whose index is not a number (NaN input, or an infinite range) lands
// in no bin there (a typed-array store at index NaN does nothing), so it is skipped here.  Counts per block in shared
// memory, then added to 64-bit global counters.
constexpr int HIST_MAX_BINS = 4096;
__global__ void __launch_bounds__(256) histogram_f32_kernel(const float* __restrict__ x, int64_t n, double range_min, double scale,
                                                            int num_bins, unsigned long long* __restrict__ bins) {
  __shared__ unsigned int local[HIST_MAX_BINS];
  for (int i = threadIdx.x; i < num_bins; i += blockDim.x) local[i] = 0u;
  __syncthreads();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const double top = (double)(num_bins - 1);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const double raw = ((double)__ldcs(x + i) - range_min) * scale;
    const double f = floor(raw);
    if (raw == raw && f >= 0.0) atomicAdd(&local[f > top ? num_bins - 1 : (int)f], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < num_bins; i += blockDim.x)
    if (local[i]) atomicAdd(bins + i, (unsigned long long)local[i]);
}

// Picks the instance of quantize_per_token_warp_kernel for a row length: vectors per lane and warps per row chosen so
// that a lane holds at most 24 vectors (128 registers or fewer) and short rows leave room for many warps per SM.
template <bool KEYS>
int launch_warp_rows(b200q_ctx* ctx, const float* x, int64_t M, int64_t K, int64_t ld_in4, int64_t ld_out4, const uint32_t* keys,
                     int8_t* q, float* scales, int qmin, int qmax) {
  const int K4 = (int)(K / 4);
  typedef void (*WarpFn)(const float*, int64_t, int, int64_t, int64_t, const uint32_t*, int8_t*, float*, float, float);
  WarpFn fn;
  int rows_per_block, threads;
  if (K4 <= 128)       { fn = quantize_per_token_warp_kernel<4, 1, 8, KEYS>;  rows_per_block = 8; threads = 256; }
  else if (K4 <= 256)  { fn = quantize_per_token_warp_kernel<8, 1, 8, KEYS>;  rows_per_block = 8; threads = 256; }
  else if (K4 <= 384)  { fn = quantize_per_token_warp_kernel<12, 1, 4, KEYS>; rows_per_block = 4; threads = 128; }
  else if (K4 <= 512)  { fn = quantize_per_token_warp_kernel<16, 1, 4, KEYS>; rows_per_block = 4; threads = 128; }
  else if (K4 <= 768)  { fn = quantize_per_token_warp_kernel<24, 1, 4, KEYS>; rows_per_block = 4; threads = 128; }
  else if (K4 <= 1024) { fn = quantize_per_token_warp_kernel<16, 2, 4, KEYS>; rows_per_block = 2; threads = 128; }
  else if (K4 <= 1536) { fn = quantize_per_token_warp_kernel<24, 2, 4, KEYS>; rows_per_block = 2; threads = 128; }
  else if (K4 <= 2048) { fn = quantize_per_token_warp_kernel<16, 4, 4, KEYS>; rows_per_block = 1; threads = 128; }
  else if (K4 <= 3072) { fn = quantize_per_token_warp_kernel<24, 4, 4, KEYS>; rows_per_block = 1; threads = 128; }
  else if (K4 <= 4096) { fn = quantize_per_token_warp_kernel<16, 8, 8, KEYS>; rows_per_block = 1; threads = 256; }
  else if (K4 <= 6144) { fn = quantize_per_token_warp_kernel<24, 8, 8, KEYS>; rows_per_block = 1; threads = 256; }
  else                 { fn = quantize_per_token_warp_kernel<16, 16, 16, KEYS>; rows_per_block = 1; threads = 512; }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((M + rows_per_block - 1) / rows_per_block));
  cfg.blockDim = dim3(threads);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->profiling ? 0 : 1;
  B200Q_CHECK_CUDA(cudaLaunchKernelEx(&cfg, fn, x, M, K4, ld_in4, ld_out4, keys, q, scales, (float)qmin, (float)qmax));
  return 0;
}
constexpr int64_t WARP_ROWS_MAX_K = 32768;   // 16 warps of 16 vectors

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// ----------------------------------------------------------------------------
// Launchers
// ----------------------------------------------------------------------------
int launch_quantize_per_token(b200q_ctx* ctx, const float* x, int64_t M, int64_t K, int8_t* q, float* scales, int qmin,
                              int qmax) {
  ProfScope prof(ctx, KK_QUANT_TOKEN);
  if (M == 0 || K == 0) {
    return 0;
  }
  const bool vec = (K % 4 == 0) && aligned16(x) && ((reinterpret_cast<uintptr_t>(q) & 3u) == 0) && (K / 4 <= 8 * 1024);
  // Teams of warps per row, the row in registers straight from global memory: rows of 128 to 16384 elements.
  const bool warp_rows = vec && K >= 128 && K <= WARP_ROWS_MAX_K && (ctx->quant_variant == 3 || ctx->quant_variant == 0);
  // Otherwise rows of up to 16 KB are staged through shared memory by bulk copies; longer rows stay in registers.
  const bool staged = vec && !warp_rows && ctx->quant_variant != 1 && ctx->quant_variant != 3 && K * 4 <= 16384 && M >= 64;
  if (warp_rows) {
    if (int e = launch_warp_rows<false>(ctx, x, M, K, K / 4, K / 4, nullptr, q, scales, qmin, qmax)) return e;
  } else if (staged) {
    const int K4 = (int)(K / 4);
    const int64_t row_bytes = K * 4;
    int rows_per_chunk = (int)(8192 / row_bytes);
    if (rows_per_chunk < 1) rows_per_chunk = 1;
    const int64_t chunk_bytes = row_bytes * rows_per_chunk;
    int slots = (int)((196 * 1024) / chunk_bytes);
    if (slots > QT_MAX_SLOTS) slots = QT_MAX_SLOTS;
    const size_t smem = (size_t)slots * chunk_bytes;
    // Rows of 8, 12 and 16 KB go through the register-resident form (one row per slot there).
    typedef void (*StagedFn)(const float*, int64_t, int, int, int, int8_t*, float*, float, float, uint32_t*, unsigned long long);
    StagedFn fn = quantize_per_token_staged_kernel<QT_CONSUMER_WARPS, 0>;
    int consumer_warps = QT_CONSUMER_WARPS, ready_bit = 0;
    if (rows_per_chunk == 1 && ctx->quant_variant != 2) {   // variants 0 and 4
      if (K4 == 32 * 32) { fn = quantize_per_token_staged_kernel<11, 32>; consumer_warps = 11; ready_bit = 1; }
      else if (K4 == 32 * 24) { fn = quantize_per_token_staged_kernel<14, 24>; consumer_warps = 14; ready_bit = 2; }
      else if (K4 == 32 * 16) { fn = quantize_per_token_staged_kernel<14, 16>; consumer_warps = 14; ready_bit = 3; }
    }
    if (!(ctx->quant_staged_ready & (1u << ready_bit))) {
      B200Q_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      ctx->quant_staged_ready |= 1u << ready_bit;
    }
    const int64_t num_chunks = (M + rows_per_chunk - 1) / rows_per_chunk;
    const unsigned blocks = (unsigned)(num_chunks < ctx->sm_count ? num_chunks : ctx->sm_count);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(32 * (consumer_warps + 1));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->profiling ? 0 : 1;   // with profiling on an event separates the kernels anyway
    B200Q_CHECK_CUDA(cudaLaunchKernelEx(&cfg, fn, x, M, K4, rows_per_chunk, slots, q, scales,
                                        (float)qmin, (float)qmax, ctx->status_dev,
                                        (unsigned long long)(ctx->wait_limit_s * 1e9)));
  } else if (vec) {
    const int K4 = (int)(K / 4);
    int G = 32;
    while (G < 1024 && (K4 + G - 1) / G > 4) G <<= 1;
    const int vpt_needed = (K4 + G - 1) / G;
    const int threads = G < 256 ? 256 : G;
    const int rows_per_block = threads / G;
    typedef void (*Kern)(const float*, int64_t, int, int, int8_t*, float*, float, float);
    const bool small = threads <= 256;
    const Kern kern = vpt_needed <= 1   ? (small ? quantize_per_token_vec_kernel<1, 256> : quantize_per_token_vec_kernel<1, 1024>)
                      : vpt_needed <= 2 ? (small ? quantize_per_token_vec_kernel<2, 256> : quantize_per_token_vec_kernel<2, 1024>)
                      : vpt_needed <= 4 ? (small ? quantize_per_token_vec_kernel<4, 256> : quantize_per_token_vec_kernel<4, 1024>)
                                        : (small ? quantize_per_token_vec_kernel<8, 256> : quantize_per_token_vec_kernel<8, 1024>);
    int per_sm = 1;
    B200Q_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, threads, 0));
    if (per_sm < 1) per_sm = 1;
    int64_t blocks = (M + rows_per_block - 1) / rows_per_block;
    const int64_t resident = (int64_t)ctx->sm_count * per_sm;
    if (blocks > resident) blocks = resident;
    kern<<<(unsigned)blocks, threads, 0, ctx->stream>>>(x, M, K4, G, q, scales, (float)qmin, (float)qmax);
  } else {
    const unsigned blocks = (unsigned)(M < (int64_t)ctx->sm_count * 8 ? M : (int64_t)ctx->sm_count * 8);
    quantize_per_token_generic_kernel<<<blocks, 256, 0, ctx->stream>>>(x, M, K, q, scales, (float)qmin, (float)qmax);
  }
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_dequantize_per_token(b200q_ctx* ctx, const int8_t* q, const float* scales, int64_t M, int64_t K, float* y) {
  ProfScope prof(ctx, KK_DEQUANT_TOKEN);
  if (M == 0 || K == 0) return 0;
  const bool vec = (K % 4 == 0) && aligned16(y) && ((reinterpret_cast<uintptr_t>(q) & 3u) == 0) && M < (1ll << 31);
  if (vec) {
    const int K4 = (int)(K / 4);
    constexpr int VPT = 4;
    const int per_block = 256 * VPT;
    dim3 grid((unsigned)M, (unsigned)((K4 + per_block - 1) / per_block));
    dequantize_per_token_vec_kernel<VPT><<<grid, 256, 0, ctx->stream>>>(q, scales, M, K4, y);
  } else {
    const unsigned blocks = (unsigned)(M < (int64_t)ctx->sm_count * 8 ? M : (int64_t)ctx->sm_count * 8);
    dequantize_per_token_generic_kernel<<<blocks, 256, 0, ctx->stream>>>(q, scales, M, K, y);
  }
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

static unsigned flat_blocks(b200q_ctx* ctx, int64_t work_items) {
  int64_t b = (work_items + 255) / 256;
  int64_t cap = (int64_t)ctx->sm_count * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

int launch_quantize_static(b200q_ctx* ctx, const float* x, int64_t n, double scale, int zp, int dst_kind, void* q) {
  ProfScope prof(ctx, KK_QUANT_STATIC);
  if (n == 0) return 0;
  const float inv = (float)(1.0 / scale);
  const float a = inv < 0 ? -inv : inv;
  const int exact_only = !(a >= 1.17549435e-38f && a <= 3.402823466e38f) || zp != 0;
  const float qmin = dst_kind == 1 ? 0.0f : -128.0f, qmax = dst_kind == 1 ? 255.0f : 127.0f;
  const int vec_ok = aligned16(x) && ((reinterpret_cast<uintptr_t>(q) & 3u) == 0);
  quantize_static_kernel<<<flat_blocks(ctx, (n + 3) / 4), 256, 0, ctx->stream>>>(x, n, scale, inv, (float)zp, exact_only, qmin,
                                                                                   qmax, (int8_t*)q, vec_ok);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_dequantize_static(b200q_ctx* ctx, const void* q, int src_kind, int64_t n, double scale, int zp, float* y) {
  ProfScope prof(ctx, KK_DEQUANT_STATIC);
  if (n == 0) return 0;
  if (src_kind == 2) {
    dequantize_static_i32_kernel<<<flat_blocks(ctx, n), 256, 0, ctx->stream>>>((const int32_t*)q, n, scale, (float)zp, y);
  } else {
    const int vec_ok = aligned16(y) && ((reinterpret_cast<uintptr_t>(q) & 3u) == 0);
    dequantize_static_8_kernel<<<flat_blocks(ctx, (n + 3) / 4), 256, 0, ctx->stream>>>((const uint8_t*)q, n, scale, (float)zp,
                                                                                         src_kind, y, vec_ok);
  }
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_quantize_weights(b200q_ctx* ctx, const float* w, int64_t N, int64_t K, int layout, int qmin, int qmax, int8_t* qw,
                            float* scales32, double* scales64) {
  ProfScope prof(ctx, KK_WEIGHTS);
  if (N == 0 || K == 0) return 0;
  double* s64 = scales64;
  if (!s64) {
    if (ws_reserve(ctx, ctx->ws_acc, (size_t)N * sizeof(double))) return 1;
    s64 = (double*)ctx->ws_acc.ptr;
  }
  const unsigned rb = (unsigned)(N < (int64_t)ctx->sm_count * 8 ? N : (int64_t)ctx->sm_count * 8);
  weight_range_kernel<<<rb, 256, 0, ctx->stream>>>(w, N, K, layout, s64, scales32);
  dim3 grid((unsigned)((K + 31) / 32), (unsigned)((N + 31) / 32));
  weight_quantize_kernel<<<grid, 256, 0, ctx->stream>>>(w, N, K, layout, s64, (float)qmin, (float)qmax, qw);
  ctx->launches += 2;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_row_range(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld, float* mn, float* mx) {
  ProfScope prof(ctx, KK_QUANT_TOKEN);
  if (M == 0) return 0;
  const unsigned blocks = (unsigned)(M < (int64_t)ctx->sm_count * 8 ? M : (int64_t)ctx->sm_count * 8);
  row_range_kernel<<<blocks, 256, 0, ctx->stream>>>(y, M, N, ld, mn, mx);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_quantize_rows_with_range(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld_in, const float* mn,
                                    const float* mx, int8_t* q, int64_t ld_out, float* scales, int qmin, int qmax) {
  ProfScope prof(ctx, KK_QUANT_TOKEN);
  if (M == 0 || N == 0) return 0;
  const unsigned blocks = (unsigned)(M < (int64_t)ctx->sm_count * 8 ? M : (int64_t)ctx->sm_count * 8);
  quantize_rows_with_range_kernel<<<blocks, 256, 0, ctx->stream>>>(y, M, N, ld_in, mn, mx, q, ld_out, scales, (float)qmin, (float)qmax);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_quantize_rows_with_keys(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld_in, const uint32_t* keys,
                                   int8_t* q, int64_t ld_out, float* scales, int qmin, int qmax) {
  ProfScope prof(ctx, KK_QUANT_TOKEN);
  if (M == 0 || N == 0) return 0;
  const unsigned blocks = (unsigned)(M < (int64_t)ctx->sm_count * 8 ? M : (int64_t)ctx->sm_count * 8);
  const bool vec = N % 4 == 0 && ld_in % 4 == 0 && ld_out % 4 == 0 && aligned16(y) && (reinterpret_cast<uintptr_t>(q) & 3u) == 0 &&
                   N / 4 < (1ll << 31);
  if (vec && N >= 128 && N <= WARP_ROWS_MAX_K && ctx->quant_variant != 1) {
    if (int e = launch_warp_rows<true>(ctx, y, M, N, ld_in / 4, ld_out / 4, keys, q, scales, qmin, qmax)) return e;
  } else if (vec) {
    const int N4 = (int)(N / 4);
    if (N4 >= 4 * 256)
      quantize_rows_with_keys_vec_kernel<4><<<blocks, 256, 0, ctx->stream>>>(y, M, N4, ld_in, keys, q, ld_out, scales, (float)qmin, (float)qmax);
    else
      quantize_rows_with_keys_vec_kernel<1><<<blocks, 256, 0, ctx->stream>>>(y, M, N4, ld_in, keys, q, ld_out, scales, (float)qmin, (float)qmax);
  } else {
    quantize_rows_with_keys_kernel<<<blocks, 256, 0, ctx->stream>>>(y, M, N, ld_in, keys, q, ld_out, scales, (float)qmin, (float)qmax);
  }
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_range_to_keys(b200q_ctx* ctx, const float* mn, const float* mx, int64_t M, uint32_t* keys) {
  if (M == 0) return 0;
  range_to_keys_kernel<<<(unsigned)((M + 255) / 256), 256, 0, ctx->stream>>>(mn, mx, M, keys);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_histogram_f32(b200q_ctx* ctx, const float* x, int64_t n, double range_min, double range_max, int num_bins,
                         unsigned long long* bins) {
  ProfScope prof(ctx, KK_WEIGHTS);
  B200Q_REQUIRE(num_bins >= 1 && num_bins <= HIST_MAX_BINS, "histogram: %d bins is outside [1, %d]", num_bins, HIST_MAX_BINS);
  if (n == 0) return 0;
  const double range = range_max - range_min;
  if (!(range > 0.0)) return 0;                       // HistogramCollector.update returns before binning (calibration.ts:62-63)
  const double scale = (double)num_bins / range;
  histogram_f32_kernel<<<flat_blocks(ctx, n / 8 + 1), 256, 0, ctx->stream>>>(x, n, range_min, scale, num_bins, bins);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_transpose_i8(b200q_ctx* ctx, const int8_t* src_kn, int64_t K, int64_t N, int8_t* dst_nk) {
  ProfScope prof(ctx, KK_WEIGHTS);
  if (N == 0 || K == 0) return 0;
  dim3 grid((unsigned)((K + 31) / 32), (unsigned)((N + 31) / 32));
  transpose_i8_kernel<<<grid, 256, 0, ctx->stream>>>(src_kn, K, N, dst_nk);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_minmax_observe(b200q_ctx* ctx, const float* x, int64_t n, float* state) {
  ProfScope prof(ctx, KK_QUANT_STATIC);
  if (n == 0) return 0;
  int64_t blocks = (n / 4 + 255) / 256;
  const int64_t cap = (int64_t)ctx->sm_count * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  minmax_observe_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, n, state);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200q
