// f32 pieces of a transformer block around the int8 linears: embedding gather, LayerNorm with the next linear's
// per-token quantization fused into its tail, causal scaled-dot-product attention, residual add.
//
// What they compute (reference, paths inside the reference project):
//   embedding    src/nn/functional/embedding.ts:6-11 (index_select of table rows), positions added as the GPT-2 fixture
//                does (tests/_utils/gpt2_model.js:11-13)
//   layer norm   src/compiler/passes/decompose/decomposition_pass.ts:232-260: mean, centred values, mean of their
//                squares, rsqrt(var + eps), gamma, beta -- every step a binary32 operation
//   attention    src/nn/functional/attention.ts:42-74: matmul(q, k^T) * 1/sqrt(E), additive mask (0 / -Infinity with
//                j <= i + S - L), softmax over the keys (decomposition_pass.ts:156-174: max, exp, sum, divide), matmul with v
//   residual     ops.add in src/nn/modules/transformer.ts:144-152
// These are floating-point kernels: their results are checked to the stated tolerance (1e-5 of the output's largest
// magnitude), not bit for bit -- the reference's own summation order depends on which of its lowerings runs.  The
// int8 codes and scales LayerNorm emits ARE exact: they are the per-token quantization (same rules and fallbacks as
// quant_kernels.cu) of exactly the binary32 values the kernel would store as its f32 output.
#include "common.cuh"
#include "kernels.cuh"
#include "quant_math.cuh"

namespace b200q {

namespace {

// ---------------------------------------------------------------------------
// Embedding: out[m, :] = table[tokens[m], :] (+ pos_table[m % S, :]).  128-bit copies; a token outside the table
// sets STATUS_BAD_INDEX and yields a row of zeros.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embedding_kernel(const float* __restrict__ table, const int32_t* __restrict__ tokens,
                                                        const float* __restrict__ pos_table, int64_t M, int D4, int64_t V, int S,
                                                        float* __restrict__ out, uint32_t* status) {
  const int64_t total = M * D4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / D4;
    const int c = (int)(i - m * D4);
    const int64_t t = tokens[m];
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (t >= 0 && t < V) {
      v = __ldg(reinterpret_cast<const float4*>(table) + t * D4 + c);
      if (pos_table != nullptr) {
        const float4 p = __ldg(reinterpret_cast<const float4*>(pos_table) + (m % S) * D4 + c);
        v.x = __fadd_rn(v.x, p.x); v.y = __fadd_rn(v.y, p.y); v.z = __fadd_rn(v.z, p.z); v.w = __fadd_rn(v.w, p.w);
      }
    } else if (c == 0) {
      atomicOr(status, STATUS_BAD_INDEX);
    }
    __stcs(reinterpret_cast<float4*>(out) + i, v);
  }
}

__global__ void __launch_bounds__(256) add_f32_kernel(const float4* __restrict__ a, const float4* __restrict__ b, int64_t n4,
                                                      float4* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 x = __ldcs(a + i), y = __ldcs(b + i);
    __stcs(out + i, make_float4(__fadd_rn(x.x, y.x), __fadd_rn(x.y, y.y), __fadd_rn(x.z, y.z), __fadd_rn(x.w, y.w)));
  }
}

// ---------------------------------------------------------------------------
// LayerNorm over the last axis + per-token quantization of the result.  One warp per row, the row in registers
// (VPT float4 per lane): x (+ residual) -> mean -> centred -> variance -> normalised, gamma, beta -> range -> codes.
// Optional outputs: the sum x + residual (the block needs it again for its next residual add) and the normalised f32
// values themselves.  Reads 4 (or 8) bytes and writes 1 byte per element when only the codes are wanted.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ double ln_row_scale(float mn_f, float mx_f) {   // quantization_types.ts:308-316, 271-275
  double mn = (double)mn_f, mx = (double)mx_f;
  if (!isfinite(mn)) mn = -1.0;
  if (!isfinite(mx)) mx = 1.0;
  if (mn == mx) { mn -= 0.5; mx += 0.5; }
  const double absmax = fmax(fabs(mn), fabs(mx));
  const double s = absmax / 127.0;
  return (s == 0.0 || s != s) ? 1e-10 : s;
}

// Rows of up to 768 elements fit 80 registers without spills: three blocks per SM instead of two.
template <int VPT>
__global__ void __launch_bounds__(256, VPT <= 6 ? 3 : 2) layernorm_quantize_kernel(const float* __restrict__ x, const float* __restrict__ residual,
                                                                  const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                  float eps, int64_t M, int D4, float* __restrict__ sum_out,
                                                                  float* __restrict__ y_out, int8_t* __restrict__ q_out,
                                                                  float* __restrict__ scales_out) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const float inv_d = 1.0f / (float)(D4 * 4);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the linear that follows may start its set-up early
  for (int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < M; row += warps) {
    const float4* xr = reinterpret_cast<const float4*>(x) + row * D4;
    float4 v[VPT];
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int c = lane + 32 * j;
      v[j] = (c < D4) ? __ldcs(xr + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (residual != nullptr) {
      const float4* rr = reinterpret_cast<const float4*>(residual) + row * D4;
#pragma unroll
      for (int j = 0; j < VPT; j++) {
        const int c = lane + 32 * j;
        if (c < D4) {
          const float4 r = __ldcs(rr + c);
          v[j].x = __fadd_rn(v[j].x, r.x); v[j].y = __fadd_rn(v[j].y, r.y); v[j].z = __fadd_rn(v[j].z, r.z); v[j].w = __fadd_rn(v[j].w, r.w);
        }
      }
      if (sum_out != nullptr) {
        float4* so = reinterpret_cast<float4*>(sum_out) + row * D4;
#pragma unroll
        for (int j = 0; j < VPT; j++) {
          const int c = lane + 32 * j;
          if (c < D4) so[c] = v[j];
        }
      }
    }
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; j++) s += (v[j].x + v[j].y) + (v[j].z + v[j].w);   // dead vectors are zero
    const float mean = warp_sum(s) * inv_d;
    float sq = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int c = lane + 32 * j;
      if (c < D4) {
        v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
        sq += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
      }
    }
    const float var = warp_sum(sq) * inv_d;
    const float rstd = 1.0f / sqrtf(var + eps);
    float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000), poison = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int c = lane + 32 * j;
      if (c < D4) {
        const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + c), b = __ldg(reinterpret_cast<const float4*>(beta) + c);
        v[j].x = __fadd_rn(__fmul_rn(__fmul_rn(v[j].x, rstd), g.x), b.x);
        v[j].y = __fadd_rn(__fmul_rn(__fmul_rn(v[j].y, rstd), g.y), b.y);
        v[j].z = __fadd_rn(__fmul_rn(__fmul_rn(v[j].z, rstd), g.z), b.z);
        v[j].w = __fadd_rn(__fmul_rn(__fmul_rn(v[j].w, rstd), g.w), b.w);
        mn = fminf(fminf(mn, v[j].x), fminf(fminf(v[j].y, v[j].z), v[j].w));   // NaN operands are dropped, as the reference's
        mx = fmaxf(fmaxf(mx, v[j].x), fmaxf(fmaxf(v[j].y, v[j].z), v[j].w));   // strict comparisons do
        // ... so a NaN (or infinite) element of this lane has to be noticed separately: 0 * y is NaN exactly then
        poison = fmaf(v[j].x, 0.0f, fmaf(v[j].y, 0.0f, fmaf(v[j].z, 0.0f, fmaf(v[j].w, 0.0f, poison))));
      }
    }
    if (y_out != nullptr) {
      float4* yo = reinterpret_cast<float4*>(y_out) + row * D4;
#pragma unroll
      for (int j = 0; j < VPT; j++) {
        const int c = lane + 32 * j;
        if (c < D4) yo[c] = v[j];
      }
    }
    if (q_out == nullptr) continue;   // uniform
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    // Per-token codes of the normalised row: same rules as the standalone quantize kernels.  An ordinary row
    // (finite, not constant) takes the lean packed encode -- its elements are finite and |t| <= 127 (1 + 2^-23), so a
    // tie is the only thing that can go wrong: a cheap test with the worst-case margin first, the per-element test
    // only if that trips, the exact binary64 path only if that one does.
    const float absmax = fmaxf(fabsf(mn), fabsf(mx));
    const float inv = __fdiv_rn(127.0f, absmax);
    const float a_inv = fabsf(inv);
    const bool exact_only = !((mn < mx) && absmax <= 3.402823466e38f && a_inv >= 1.17549435e-38f && a_inv <= 3.402823466e38f);
    uint32_t words[VPT];
    bool exact = exact_only || (poison != poison);   // per lane: the exact path is right for every element
    if (!exact) {
      const uint64_t inv2 = f2_pack(inv, inv), magic2 = f2_pack(12582912.0f, 12582912.0f);
      float far = 0.0f;
#pragma unroll
      for (int j = 0; j < VPT; j++) words[j] = pack4_fast_lean(v[j], inv2, magic2, far);   // dead vectors are zero: harmless
      if (far >= 0.49993920f) {                                   // 0.5 - 127.5 * 2^-21
        int tie = 0;
#pragma unroll
        for (int j = 0; j < VPT; j++) {
          (void)quantize_fast_bounded(v[j].x, inv, tie); (void)quantize_fast_bounded(v[j].y, inv, tie);
          (void)quantize_fast_bounded(v[j].z, inv, tie); (void)quantize_fast_bounded(v[j].w, inv, tie);
        }
        exact = tie >= 0x3f000000;
      }
    }
    if (exact) {   // rare: a tie, a non-finite element, an odd row
      const double sd = ln_row_scale(mn, mx);
#pragma unroll
      for (int j = 0; j < VPT; j++)
        words[j] = pack_codes(quantize_exact_p(v[j].x, sd, -127.0f, 127.0f), quantize_exact_p(v[j].y, sd, -127.0f, 127.0f),
                              quantize_exact_p(v[j].z, sd, -127.0f, 127.0f), quantize_exact_p(v[j].w, sd, -127.0f, 127.0f));
    }
    uint32_t* qr = reinterpret_cast<uint32_t*>(q_out) + row * D4;
#pragma unroll
    for (int j = 0; j < VPT; j++) {
      const int c = lane + 32 * j;
      if (c < D4) qr[c] = words[j];
    }
    if (lane == 0) scales_out[row] = exact_only ? (float)ln_row_scale(mn, mx) : __fdiv_rn(absmax, 127.0f);
  }
}

// ---------------------------------------------------------------------------
// Scaled-dot-product attention in binary32, head dimension 64, optional causal mask.
// One block per (batch, head, 64 query rows); key/value tiles of 64 rows pass through shared memory; every thread
// owns a 4x4 patch of the 64x64 score tile and of the 64x64 output tile;
// running max / sum per row (the softmax is rescaled tile by tile, so no [S,S] matrix is ever stored).
// The transposed tiles (Q and K by feature, P by key) are unpadded and XOR-swizzled at float4 granularity -- slot
// (column / 4) ^ ((row / 4) & 7) -- which keeps both their scalar transposing stores and their float4 reads at the
// minimum number of shared-memory wavefronts.  Rows of q, k, v and out are addressed as base + (b*S + s)*ld + h*64,
// which reads the projections where the linears wrote them.
// ---------------------------------------------------------------------------
// exp through the hardware base-2 exponential: relative error about 2^-22, far inside the 1e-5 bar of these kernels.
__device__ __forceinline__ float fast_exp(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x * 1.4426950408889634f));
  return r;
}

constexpr int AT = 64;     // key tile = head dimension

// element (row, col) of a [rows][LD] tile whose float4 slots are swizzled by the row
template <int LD>
__device__ __forceinline__ int swz(int row, int col) {
  return row * LD + ((((col >> 2) ^ ((row >> 2) & 7)) << 2) | (col & 3));
}

__global__ void __launch_bounds__(256, 3) sdpa_f32_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                       const float* __restrict__ v, float* __restrict__ out, int64_t ld_q,
                                                       int64_t ld_k, int64_t ld_v, int64_t ld_o, int H, int S, float scale, int causal) {
  extern __shared__ __align__(16) float sm[];
  float* Qt = sm;                  // [d][query row], swizzled
  float* Kt = Qt + AT * AT;        // [d][key row], swizzled
  float* Vs = Kt + AT * AT;        // [key row][d]
  float* Pt = Vs + AT * AT;        // [key row][query row], swizzled
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int b = blockIdx.y / H, h = blockIdx.y - b * H;
  // Causal work grows with the query tile: the heaviest tiles are scheduled first.
  const int qt = causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;
  const int i0 = qt * AT;
  const int64_t row_base = (int64_t)b * S;
  const float ninf = __int_as_float(0xff800000);

  for (int idx = tid; idx < AT * 16; idx += 256) {
    const int r = idx >> 4, d4 = idx & 15;
    float4 val = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (i0 + r < S) val = __ldg(reinterpret_cast<const float4*>(q + (row_base + i0 + r) * ld_q + h * AT) + d4);
    Qt[swz<AT>(d4 * 4 + 0, r)] = val.x; Qt[swz<AT>(d4 * 4 + 1, r)] = val.y; Qt[swz<AT>(d4 * 4 + 2, r)] = val.z; Qt[swz<AT>(d4 * 4 + 3, r)] = val.w;
  }
  float o[4][4], m[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    m[i] = ninf; l[i] = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) o[i][j] = 0.0f;
  }
  const int ntiles = causal ? (qt + 1) : ((S + AT - 1) / AT);
  for (int kt = 0; kt < ntiles; kt++) {
    const int j0 = kt * AT;
    __syncthreads();   // the previous tile's readers are done (and, first time round, Qt is complete after the next one)
    for (int idx = tid; idx < AT * 16; idx += 256) {
      const int r = idx >> 4, d4 = idx & 15;
      float4 kv = make_float4(0.0f, 0.0f, 0.0f, 0.0f), vv = kv;
      if (j0 + r < S) {
        kv = __ldg(reinterpret_cast<const float4*>(k + (row_base + j0 + r) * ld_k + h * AT) + d4);
        vv = __ldg(reinterpret_cast<const float4*>(v + (row_base + j0 + r) * ld_v + h * AT) + d4);
      }
      Kt[swz<AT>(d4 * 4 + 0, r)] = kv.x; Kt[swz<AT>(d4 * 4 + 1, r)] = kv.y; Kt[swz<AT>(d4 * 4 + 2, r)] = kv.z; Kt[swz<AT>(d4 * 4 + 3, r)] = kv.w;
      *reinterpret_cast<float4*>(&Vs[r * AT + d4 * 4]) = vv;
    }
    __syncthreads();
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) s[i][j] = 0.0f;
#pragma unroll 8
    for (int d = 0; d < AT; d++) {
      const float4 a = *reinterpret_cast<const float4*>(&Qt[swz<AT>(d, ty * 4)]);
      const float4 c = *reinterpret_cast<const float4*>(&Kt[swz<AT>(d, tx * 4)]);
      const float av[4] = {a.x, a.y, a.z, a.w}, cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) s[i][j] = fmaf(av[i], cv[j], s[i][j]);
    }
    float alpha[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int qi = i0 + ty * 4 + i;
      float rmax = ninf;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const int kj = j0 + tx * 4 + j;
        float sv = s[i][j] * scale;
        if (kj >= S || (causal && kj > qi)) sv = ninf;
        s[i][j] = sv;
        rmax = fmaxf(rmax, sv);
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, off));
      const float m_new = fmaxf(m[i], rmax);
      const bool empty = m_new == ninf;                 // nothing unmasked in this row so far
      alpha[i] = empty ? 1.0f : fast_exp(m[i] - m_new);     // exp(-inf) = 0 when the row had nothing before
      float rsum = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float p = empty ? 0.0f : fast_exp(s[i][j] - m_new);
        s[i][j] = p;
        rsum += p;
      }
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, off);
      l[i] = l[i] * alpha[i] + rsum;
      m[i] = m_new;
#pragma unroll
      for (int j = 0; j < 4; j++) o[i][j] *= alpha[i];
    }
#pragma unroll
    for (int j = 0; j < 4; j++)
      *reinterpret_cast<float4*>(&Pt[swz<AT>(tx * 4 + j, ty * 4)]) = make_float4(s[0][j], s[1][j], s[2][j], s[3][j]);
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < AT; c++) {
      const float4 p = *reinterpret_cast<const float4*>(&Pt[swz<AT>(c, ty * 4)]);
      const float4 w = *reinterpret_cast<const float4*>(&Vs[c * AT + tx * 4]);
      const float pv[4] = {p.x, p.y, p.z, p.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o[i][j] = fmaf(pv[i], wv[j], o[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int qi = i0 + ty * 4 + i;
    if (qi < S) {
      const float inv_l = 1.0f / l[i];
      *reinterpret_cast<float4*>(out + (row_base + qi) * ld_o + h * AT + tx * 4) =
          make_float4(o[i][0] * inv_l, o[i][1] * inv_l, o[i][2] * inv_l, o[i][3] * inv_l);
    }
  }
}

// ---------------------------------------------------------------------------
// The same attention on the tensor cores with three-way tf32 products.
// A binary32 number x is split into hi = tf32(x) and lo = tf32(x - hi); a*b ~= a_hi*b_hi + a_hi*b_lo + a_lo*b_hi drops
// only the lo*lo term (2^-22 relative), and the products accumulate in binary32 -- which keeps the result inside
// the 1e-5 bar that a single tf32 product (2^-11) would miss by two orders of magnitude.
// One block = 4 warps = 64 query rows (16 per warp) of one (batch, head); key/value tiles of 64 rows are split into
// hi/lo once when they are staged in shared memory.  mma.sync m16n8k8: scores come out in the accumulator layout
// (row g / g+8, columns 2t, 2t+1 of each 8-key group); fed back as the A operand of P*V they stand for the keys in the
// order (2t, 2t+1) -> k = (t, t+4), so the V rows are fetched in that order and no shuffle is needed.
// Measured on B200 at 32 x 12 heads x 512 x 64, causal: 0.55 ms against 0.52 ms for the CUDA-core kernel above -- the
// warp-level mma.sync path does not run at tensor-core speed on this part, so this form is kept as the selectable second
// implementation (b200q_set_sdpa_variant 1) and as the layout groundwork for a tcgen05 version.
// ---------------------------------------------------------------------------
constexpr int TLD = 68;   // row length of the staged tiles (floats): fragment loads hit 32 distinct banks

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = to_tf32(x);
  lo = to_tf32(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128) sdpa_tf32x3_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                          const float* __restrict__ v, float* __restrict__ out, int64_t ld_q,
                                                          int64_t ld_k, int64_t ld_v, int64_t ld_o, int H, int S, float scale,
                                                          int causal) {
  extern __shared__ __align__(16) float sm[];
  uint32_t(*Khi)[TLD] = reinterpret_cast<uint32_t(*)[TLD]>(sm);                   // [key][d]
  uint32_t(*Klo)[TLD] = reinterpret_cast<uint32_t(*)[TLD]>(sm + AT * TLD);
  uint32_t(*Vhi)[TLD] = reinterpret_cast<uint32_t(*)[TLD]>(sm + 2 * AT * TLD);    // [key][d]
  uint32_t(*Vlo)[TLD] = reinterpret_cast<uint32_t(*)[TLD]>(sm + 3 * AT * TLD);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int b = blockIdx.y / H, h = blockIdx.y - b * H;
  const int qt = causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;   // heaviest causal tiles first
  const int i0 = qt * AT;
  const int64_t row_base = (int64_t)b * S;
  const float ninf = __int_as_float(0xff800000);
  const int r_lo = i0 + warp * 16 + g, r_hi = r_lo + 8;   // the two query rows this thread holds pieces of

  // Q fragments (scaled), split once: A operand of step kk covers d = kk*8 .. kk*8+7.
  uint32_t qh[8][4], ql[8][4];
  {
    const float* q0 = q + (row_base + (r_lo < S ? r_lo : 0)) * ld_q + h * AT;
    const float* q1 = q + (row_base + (r_hi < S ? r_hi : 0)) * ld_q + h * AT;
#pragma unroll
    for (int kk = 0; kk < 8; kk++) {
      const float x0 = (r_lo < S) ? __ldg(q0 + kk * 8 + t) * scale : 0.0f, x1 = (r_hi < S) ? __ldg(q1 + kk * 8 + t) * scale : 0.0f;
      const float x2 = (r_lo < S) ? __ldg(q0 + kk * 8 + t + 4) * scale : 0.0f, x3 = (r_hi < S) ? __ldg(q1 + kk * 8 + t + 4) * scale : 0.0f;
      split_tf32(x0, qh[kk][0], ql[kk][0]);
      split_tf32(x1, qh[kk][1], ql[kk][1]);
      split_tf32(x2, qh[kk][2], ql[kk][2]);
      split_tf32(x3, qh[kk][3], ql[kk][3]);
    }
  }
  float o[8][4];
#pragma unroll
  for (int n = 0; n < 8; n++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[n][e] = 0.0f;
  float m0 = ninf, m1 = ninf, l0 = 0.0f, l1 = 0.0f;

  const int ntiles = causal ? (qt + 1) : ((S + AT - 1) / AT);
  for (int kt = 0; kt < ntiles; kt++) {
    const int j0 = kt * AT;
    __syncthreads();   // the previous tile's readers are done
    for (int idx = tid; idx < AT * 16; idx += 128) {
      const int r = idx >> 4, d4 = idx & 15;
      float4 kv = make_float4(0.0f, 0.0f, 0.0f, 0.0f), vv = kv;
      if (j0 + r < S) {
        kv = __ldg(reinterpret_cast<const float4*>(k + (row_base + j0 + r) * ld_k + h * AT) + d4);
        vv = __ldg(reinterpret_cast<const float4*>(v + (row_base + j0 + r) * ld_v + h * AT) + d4);
      }
      uint4 hi, lo;
      split_tf32(kv.x, hi.x, lo.x); split_tf32(kv.y, hi.y, lo.y); split_tf32(kv.z, hi.z, lo.z); split_tf32(kv.w, hi.w, lo.w);
      *reinterpret_cast<uint4*>(&Khi[r][d4 * 4]) = hi;
      *reinterpret_cast<uint4*>(&Klo[r][d4 * 4]) = lo;
      split_tf32(vv.x, hi.x, lo.x); split_tf32(vv.y, hi.y, lo.y); split_tf32(vv.z, hi.z, lo.z); split_tf32(vv.w, hi.w, lo.w);
      *reinterpret_cast<uint4*>(&Vhi[r][d4 * 4]) = hi;
      *reinterpret_cast<uint4*>(&Vlo[r][d4 * 4]) = lo;
    }
    __syncthreads();

    // scores of 16 query rows x 64 keys: s[n] covers keys j0 + n*8 .. +7
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; n++) {
#pragma unroll
      for (int e = 0; e < 4; e++) s[n][e] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < 8; kk++) {
        const uint32_t bh0 = Khi[n * 8 + g][kk * 8 + t], bh1 = Khi[n * 8 + g][kk * 8 + t + 4];
        const uint32_t bl0 = Klo[n * 8 + g][kk * 8 + t], bl1 = Klo[n * 8 + g][kk * 8 + t + 4];
        mma_tf32(s[n], ql[kk], bh0, bh1);
        mma_tf32(s[n], qh[kk], bl0, bl1);
        mma_tf32(s[n], qh[kk], bh0, bh1);
      }
    }
    // mask, running max and sum per row (rows r_lo: elements 0,1; r_hi: elements 2,3)
    float mx0 = ninf, mx1 = ninf;
#pragma unroll
    for (int n = 0; n < 8; n++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int kj = j0 + n * 8 + 2 * t + (e & 1);
        const int qi = (e < 2) ? r_lo : r_hi;
        if (kj >= S || (causal && kj > qi)) s[n][e] = ninf;
      }
      mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
      mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
    }
#pragma unroll
    for (int off = 1; off <= 2; off <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const bool e0 = mn0 == ninf, e1 = mn1 == ninf;   // nothing unmasked in the row so far
    const float al0 = e0 ? 1.0f : expf(m0 - mn0), al1 = e1 ? 1.0f : expf(m1 - mn1);
    float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
    for (int n = 0; n < 8; n++) {
      s[n][0] = e0 ? 0.0f : expf(s[n][0] - mn0);
      s[n][1] = e0 ? 0.0f : expf(s[n][1] - mn0);
      s[n][2] = e1 ? 0.0f : expf(s[n][2] - mn1);
      s[n][3] = e1 ? 0.0f : expf(s[n][3] - mn1);
      sum0 += s[n][0] + s[n][1];
      sum1 += s[n][2] + s[n][3];
    }
#pragma unroll
    for (int off = 1; off <= 2; off <<= 1) {
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, off);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, off);
    }
    l0 = l0 * al0 + sum0; l1 = l1 * al1 + sum1;
    m0 = mn0; m1 = mn1;
#pragma unroll
    for (int n = 0; n < 8; n++) { o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1; }

    // O += P V: step kk uses the 8 keys of score group kk, in the order (2t -> k = t, 2t+1 -> k = t+4)
#pragma unroll
    for (int kk = 0; kk < 8; kk++) {
      uint32_t ph[4], pl[4];
      split_tf32(s[kk][0], ph[0], pl[0]);   // a0: row g,   k = t
      split_tf32(s[kk][2], ph[1], pl[1]);   // a1: row g+8, k = t
      split_tf32(s[kk][1], ph[2], pl[2]);   // a2: row g,   k = t+4
      split_tf32(s[kk][3], ph[3], pl[3]);   // a3: row g+8, k = t+4
      const int key0 = kk * 8 + 2 * t, key1 = key0 + 1;
#pragma unroll
      for (int n = 0; n < 8; n++) {
        const uint32_t bh0 = Vhi[key0][n * 8 + g], bh1 = Vhi[key1][n * 8 + g];
        const uint32_t bl0 = Vlo[key0][n * 8 + g], bl1 = Vlo[key1][n * 8 + g];
        mma_tf32(o[n], pl, bh0, bh1);
        mma_tf32(o[n], ph, bl0, bl1);
        mma_tf32(o[n], ph, bh0, bh1);
      }
    }
  }
  const float il0 = 1.0f / l0, il1 = 1.0f / l1;
#pragma unroll
  for (int n = 0; n < 8; n++) {
    if (r_lo < S)
      *reinterpret_cast<float2*>(out + (row_base + r_lo) * ld_o + h * AT + n * 8 + 2 * t) = make_float2(o[n][0] * il0, o[n][1] * il0);
    if (r_hi < S)
      *reinterpret_cast<float2*>(out + (row_base + r_hi) * ld_o + h * AT + n * 8 + 2 * t) = make_float2(o[n][2] * il1, o[n][3] * il1);
  }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

unsigned flat_grid(b200q_ctx* ctx, int64_t items, int per_block) {
  int64_t blocks = (items + per_block - 1) / per_block;
  const int64_t cap = (int64_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

}  // namespace

int launch_embedding(b200q_ctx* ctx, const float* table, const int32_t* tokens, const float* pos_table, int64_t M, int64_t D,
                     int64_t V, int64_t S, float* out) {
  ProfScope prof(ctx, KK_EMBEDDING);
  if (M == 0 || D == 0) return 0;
  B200Q_REQUIRE(D % 4 == 0 && aligned16(table) && aligned16(out) && (pos_table == nullptr || aligned16(pos_table)),
                "embedding needs a row length that is a multiple of 4 and 16-byte aligned buffers");
  B200Q_REQUIRE(pos_table == nullptr || S > 0, "embedding: a position table needs the sequence length");
  embedding_kernel<<<flat_grid(ctx, M * (D / 4), 256), 256, 0, ctx->stream>>>(table, tokens, pos_table, M, (int)(D / 4), V,
                                                                              (int)(S > 0 ? S : 1), out, ctx->status_dev);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_add_f32(b200q_ctx* ctx, const float* a, const float* b, int64_t n, float* out) {
  ProfScope prof(ctx, KK_ADD);
  if (n == 0) return 0;
  B200Q_REQUIRE(n % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(out),
                "add needs a length that is a multiple of 4 and 16-byte aligned buffers");
  add_f32_kernel<<<flat_grid(ctx, n / 4, 256), 256, 0, ctx->stream>>>(reinterpret_cast<const float4*>(a),
                                                                      reinterpret_cast<const float4*>(b), n / 4,
                                                                      reinterpret_cast<float4*>(out));
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_layernorm_quantize(b200q_ctx* ctx, const float* x, const float* residual, const float* gamma, const float* beta,
                              float eps, int64_t M, int64_t D, float* sum_out, float* y_out, int8_t* q_out, float* scales_out) {
  ProfScope prof(ctx, KK_LAYERNORM);
  if (M == 0) return 0;
  B200Q_REQUIRE(D > 0 && D % 4 == 0 && D <= 2048, "layer norm rows must be a multiple of 4 and at most 2048 elements long (got %lld)",
                (long long)D);
  B200Q_REQUIRE(aligned16(x) && aligned16(gamma) && aligned16(beta) && (residual == nullptr || aligned16(residual)) &&
                    (sum_out == nullptr || aligned16(sum_out)) && (y_out == nullptr || aligned16(y_out)) &&
                    (q_out == nullptr || (reinterpret_cast<uintptr_t>(q_out) & 3u) == 0),
                "layer norm needs 16-byte aligned f32 buffers and 4-byte aligned codes");
  B200Q_REQUIRE(q_out == nullptr || scales_out != nullptr, "layer norm: codes need a scale buffer");
  const int D4 = (int)(D / 4);
  const int vpt = (D4 + 31) / 32;
  const unsigned grid = flat_grid(ctx, M, 8);   // 8 rows (warps) per block
  typedef void (*Kern)(const float*, const float*, const float*, const float*, float, int64_t, int, float*, float*, int8_t*, float*);
  const Kern kern = vpt <= 1 ? layernorm_quantize_kernel<1> : vpt <= 2 ? layernorm_quantize_kernel<2>
                    : vpt <= 3 ? layernorm_quantize_kernel<3> : vpt <= 4 ? layernorm_quantize_kernel<4>
                    : vpt <= 6 ? layernorm_quantize_kernel<6> : vpt <= 8 ? layernorm_quantize_kernel<8>
                    : vpt <= 12 ? layernorm_quantize_kernel<12> : layernorm_quantize_kernel<16>;
  kern<<<grid, 256, 0, ctx->stream>>>(x, residual, gamma, beta, eps, M, D4, sum_out, y_out, q_out, scales_out);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_sdpa_f32(b200q_ctx* ctx, const float* q, const float* k, const float* v, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                    int64_t B, int64_t H, int64_t S, int64_t Dh, float scale, int causal, float* out, int64_t ld_o) {
  ProfScope prof(ctx, KK_SDPA);
  if (B == 0 || H == 0 || S == 0) return 0;
  B200Q_REQUIRE(Dh == AT, "attention is built for a head dimension of 64 (got %lld)", (long long)Dh);
  B200Q_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && ld_q % 4 == 0 && ld_k % 4 == 0 && ld_v % 4 == 0 &&
                    ld_o % 4 == 0 && ld_q >= H * Dh && ld_k >= H * Dh && ld_v >= H * Dh && ld_o >= H * Dh,
                "attention needs 16-byte aligned buffers and row strides that are multiples of 4 and at least H * 64");
  B200Q_REQUIRE(B * H <= 65535 && S < (1 << 24), "attention: batch * heads must not exceed 65535");
  const bool umma_ok = sdpa_umma_supported(q, k, v, out, ld_q, ld_k, ld_v, ld_o, B, H, S, Dh);
  B200Q_REQUIRE(ctx->sdpa_variant != 2 || umma_ok, "attention: the tensor-core kernel does not take this shape or alignment");
  if ((ctx->sdpa_variant == 0 || ctx->sdpa_variant == 2) && umma_ok) {
    if (int e = launch_sdpa_umma(ctx, q, k, v, ld_q, ld_k, ld_v, B, H, S, scale, causal, out, ld_o)) return e;
    ctx->launches++;
    B200Q_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  const size_t smem_fma = (size_t)(4 * AT * AT) * sizeof(float), smem_mma = (size_t)4 * AT * TLD * sizeof(float);
  if (!ctx->sdpa_ready) {
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(sdpa_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_fma));
    B200Q_CHECK_CUDA(cudaFuncSetAttribute(sdpa_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma));
    ctx->sdpa_ready = true;
  }
  if (ctx->sdpa_variant == 1) {   // mma.sync with three-way tf32 products (measured slower on B200: see the kernel's comment)
    const dim3 grid((unsigned)((S + AT - 1) / AT), (unsigned)(B * H));
    sdpa_tf32x3_kernel<<<grid, 128, smem_mma, ctx->stream>>>(q, k, v, out, ld_q, ld_k, ld_v, ld_o, (int)H, (int)S, scale, causal);
  } else {
    const dim3 grid((unsigned)((S + AT - 1) / AT), (unsigned)(B * H));
    sdpa_f32_kernel<<<grid, 256, smem_fma, ctx->stream>>>(q, k, v, out, ld_q, ld_k, ld_v, ld_o, (int)H, (int)S, scale, causal);
  }
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200q
