// The two op families next to the linear path in the reference's quantization support:
//
//  * per-group quantization of a constant (GPTQ / AWQ-style INT4): QuantizationParams.fromConstantArrayPerGroup,
//    quantizeArrayPerGroup, dequantizeArrayPerGroup (src/compiler/ir/graph/quantization_types.ts:319-340, 143-162);
//  * quantized_conv with two spatial dimensions (src/compiler/ir/graph/ops/quantization.ts:156-190, lowered by
//    src/compiler/passes/lowering/rules/quantization.ts:44-62 over the loop nest of lowering_registry.ts:335-449):
//    int8 x int8 -> int32, zero-points subtracted tap by tap, a tap outside the input adds 0.
//
// The convolution runs as a contraction: a gather kernel lays the receptive fields out as the rows of an int8 matrix
// ([N*OH*OW, C/groups*KH*KW], padded to a multiple of 16 columns, padding taps holding the input zero-point so that
// their term vanishes), the tensor-core GEMM (with the zero-point correction terms when a zero-point is not 0) multiplies it with the
// kernel tensor read in place as [O, C/groups*KH*KW], and channel-first output is transposed out of the GEMM's
// channel-last result.  Groups are handled one contraction per group.  With a multiple of 16 channels per group the
// gather moves 16 bytes at a time from a channel-last input; a channel-first input and its kernel tensor are re-laid
// channel-last first.
#include <cstdint>

#include "common.cuh"
#include "kernels.cuh"
#include "quant_math.cuh"

namespace b200q {

namespace {

// ---------------------------------------------------------------------------------------------- per-group codes
// max(cMin, min(cMax, Math.round(x / s))) in binary64, then an Int8Array store: NaN (a NaN element, or Inf / Inf when
// the group's scale is infinite) becomes 0.
__device__ __forceinline__ int quantize_exact_g(float x, double s, float qmin, float qmax) {
  const double t = (double)x / s;
  if (t != t) return 0;
  const float r = (float)js_round_f64(t);
  return (int)fminf(fmaxf(r, qmin), qmax);
}

// One warp per group at a time: |x| maximum with the reference's comparison (a > absMax: NaN never wins), the scale in
// binary64 (absMax / bound, or 1e-10 when that is 0), then the codes: x * fl32(1 / scale) rounded by the streaming
// kernels' fast rule, and the exact binary64 division for every element the guard does not clear (near a tie, NaN,
// infinite, a scale whose reciprocal is not a normal binary32 number).  VEC: the group size is a multiple of 4 and the
// arrays are 16-byte aligned, so a lane moves four elements at a time.
template <bool VEC>
__global__ void __launch_bounds__(256) group_quantize_kernel(const float* __restrict__ x, int64_t n, int64_t group_size,
                                                             int64_t groups, double bound, float qmin, float qmax,
                                                             int8_t* __restrict__ q, double* __restrict__ scales64,
                                                             float* __restrict__ scales32) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const float limit = fminf(-qmin, qmax) + 0.49f;
  for (int64_t g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); g < groups; g += warps) {
    const int64_t start = g * group_size, end = (start + group_size < n) ? start + group_size : n;
    float am = 0.0f;
    if (VEC) {
      for (int64_t i = start + 4 * lane; i < end; i += 128) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(x + i));
        const float a[4] = {fabsf(v.x), fabsf(v.y), fabsf(v.z), fabsf(v.w)};
#pragma unroll
        for (int e = 0; e < 4; e++)
          if (a[e] > am) am = a[e];
      }
    } else {
      for (int64_t i = start + lane; i < end; i += 32) {
        const float a = fabsf(x[i]);
        if (a > am) am = a;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float b = __shfl_xor_sync(0xffffffffu, am, o);
      if (b > am) am = b;
    }
    double s = (double)am / bound;
    if (s == 0.0) s = 1e-10;
    if (lane == 0) {
      if (scales64) scales64[g] = s;
      if (scales32) scales32[g] = (float)s;
    }
    if (!q) continue;
    const float inv = (float)(1.0 / s);
    if (VEC) {
      for (int64_t i = start + 4 * lane; i < end; i += 128) {       // the group was just read: these loads hit the cache
        const float4 v = __ldg(reinterpret_cast<const float4*>(x + i));
        const float xv[4] = {v.x, v.y, v.z, v.w};
        int c[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
          QuantGuard guard;
          c[e] = quantize_fast(xv[e], inv, guard);
          if (guard.unsafe(limit)) c[e] = quantize_exact_g(xv[e], s, qmin, qmax);
        }
        *reinterpret_cast<uint32_t*>(q + i) = pack_codes(c[0], c[1], c[2], c[3]);
      }
    } else {
      for (int64_t i = start + lane; i < end; i += 32) {
        QuantGuard guard;
        int c = quantize_fast(x[i], inv, guard);
        if (guard.unsafe(limit)) c = quantize_exact_g(x[i], s, qmin, qmax);
        q[i] = (int8_t)c;
      }
    }
  }
}

// (q - 0) * scale[group] in binary64; the binary32 copy is that number stored to a Float32Array.
__global__ void __launch_bounds__(256) group_dequantize_kernel(const int8_t* __restrict__ q, int64_t n, int64_t group_size,
                                                               const double* __restrict__ scales64, double* __restrict__ y64,
                                                               float* __restrict__ y32) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const double v = ((double)q[i] - 0.0) * scales64[i / group_size];
    if (y64) y64[i] = v;
    if (y32) y32[i] = (float)v;
  }
}

// ---------------------------------------------------------------------------------------------- convolution
struct ConvGeom {
  int64_t N, C, H, W, O, KH, KW, OH, OW;
  int sh, sw, pt, pl, dh, dw;
  int groups, zp_in, zp_ker, layout;   // layout 0: NCHW / OIHW, 1: NHWC / OHWI
  int64_t Cg, Og, Kg, Kp;              // channels per group (in, out), taps per output of a group, padded to 16
};

// Rows of the gathered matrix for group g: row m = (n, oh, ow), column k in the kernel tensor's own order
// ((ic, kh, kw) channel-first, (kh, kw, ic) channel-last).  A thread writes 16 consecutive columns of one row.
__global__ void __launch_bounds__(256) conv_gather_kernel(const int8_t* __restrict__ in, ConvGeom p, int g, int8_t* __restrict__ a) {
  const int64_t M = p.N * p.OH * p.OW, pieces = p.Kp / 16;
  const int64_t total = M * pieces, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int64_t m = t / pieces, k0 = (t - m * pieces) * 16;
    const int64_t ow = m % p.OW, oh = (m / p.OW) % p.OH, n = m / (p.OW * p.OH);
    alignas(16) int8_t v[16];
#pragma unroll
    for (int j = 0; j < 16; j++) {
      const int64_t k = k0 + j;
      int val = p.zp_in;
      if (k < p.Kg) {
        int64_t ic, kh, kw;
        if (p.layout == 0) { kw = k % p.KW; kh = (k / p.KW) % p.KH; ic = k / (p.KW * p.KH); }
        else { ic = k % p.Cg; kw = (k / p.Cg) % p.KW; kh = k / (p.Cg * p.KW); }
        const int64_t ih = oh * p.sh + kh * p.dh - p.pt, iw = ow * p.sw + kw * p.dw - p.pl;
        if (ih >= 0 && ih < p.H && iw >= 0 && iw < p.W) {
          const int64_t c = (int64_t)g * p.Cg + ic;
          val = p.layout == 0 ? in[((n * p.C + c) * p.H + ih) * p.W + iw] : in[((n * p.H + ih) * p.W + iw) * p.C + c];
        }
      }
      v[j] = (int8_t)val;
    }
    *reinterpret_cast<uint4*>(a + m * p.Kp + k0) = *reinterpret_cast<const uint4*>(v);
  }
}

// The same rows when the input is channel-last and a group has a multiple of 16 channels: a 16-byte piece of a row is
// 16 consecutive channels of one tap, i.e. one aligned 16-byte load (or the zero-point, outside the input).
__global__ void __launch_bounds__(256) conv_gather_nhwc16_kernel(const int8_t* __restrict__ in, ConvGeom p, int g, int8_t* __restrict__ a) {
  // One thread per (output position, 16-channel piece): the position is decoded once, the taps are a plain double loop.
  const uint32_t ppt = (uint32_t)(p.Cg / 16);
  const int64_t M = p.N * p.OH * p.OW, total = M * ppt, stride = (int64_t)gridDim.x * blockDim.x;
  const uint32_t fill = 0x01010101u * (uint32_t)(uint8_t)p.zp_in;
  const uint32_t OW = (uint32_t)p.OW, OH = (uint32_t)p.OH;
  const int KH = (int)p.KH, KW = (int)p.KW, H = (int)p.H, W = (int)p.W;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const uint32_t m = (uint32_t)(t / ppt), c16 = (uint32_t)(t - (int64_t)m * ppt);
    const uint32_t ow = m % OW, mo = m / OW, oh = mo % OH, n = mo / OH;
    const int8_t* src = in + (int64_t)n * H * W * p.C + (int64_t)g * p.Cg + (int64_t)c16 * 16;
    int8_t* dst = a + (int64_t)m * p.Kp + (int64_t)c16 * 16;
    const int ih0 = (int)oh * p.sh - p.pt, iw0 = (int)ow * p.sw - p.pl;
    for (int kh = 0; kh < KH; kh++) {
      const int ih = ih0 + kh * p.dh;
      const bool row_in = ih >= 0 && ih < H;
      for (int kw = 0; kw < KW; kw++) {
        const int iw = iw0 + kw * p.dw;
        uint4 v = make_uint4(fill, fill, fill, fill);
        if (row_in && iw >= 0 && iw < W) v = __ldg(reinterpret_cast<const uint4*>(src + ((int64_t)ih * W + iw) * p.C));
        *reinterpret_cast<uint4*>(dst + (int64_t)(kh * KW + kw) * p.Cg) = v;
      }
    }
  }
}

// Batched int8 transpose: `batch` matrices [rows, cols] -> [cols, rows] (an image from channel-first to channel-last,
// an output channel's taps from (ic, kh, kw) to (kh, kw, ic) order).
__global__ void __launch_bounds__(256) conv_relay_i8_kernel(const int8_t* __restrict__ src, int64_t rows, int64_t cols,
                                                            int8_t* __restrict__ dst) {
  __shared__ int8_t tile[32][33];
  const int64_t b = blockIdx.z, r0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  src += b * rows * cols;
  dst += b * rows * cols;
  for (int j = ty; j < 32; j += 8) {
    const int64_t r = r0 + j, c = c0 + tx;
    tile[j][tx] = (r < rows && c < cols) ? src[r * cols + c] : (int8_t)0;
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int64_t c = c0 + j, r = r0 + tx;
    if (c < cols && r < rows) dst[c * rows + r] = tile[tx][j];
  }
}

// The same transpose four bytes at a time, for matrices whose extents are multiples of 4 (an image of C x H*W): a 64x64
// tile is read as words along the source rows and written as words along the destination rows.
__global__ void __launch_bounds__(256) conv_relay_i8x4_kernel(const int8_t* __restrict__ src, int64_t rows, int64_t cols,
                                                              int8_t* __restrict__ dst) {
  __shared__ uint32_t tile[64][17];     // 64 source rows x 64 columns; the pad keeps a column of words on distinct banks
  const int64_t b = blockIdx.z, r0 = (int64_t)blockIdx.y * 64, c0 = (int64_t)blockIdx.x * 64;
  src += b * rows * cols;
  dst += b * rows * cols;
  for (int i = threadIdx.x; i < 64 * 16; i += 256) {
    const int r = i >> 4, w = i & 15;
    const int64_t rr = r0 + r, cc = c0 + 4 * w;
    tile[r][w] = (rr < rows && cc < cols) ? __ldg(reinterpret_cast<const uint32_t*>(src + rr * cols + cc)) : 0u;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 16; i += 256) {
    const int c = i >> 4, w = i & 15;                   // destination row c0 + c, bytes 4w .. 4w+3 = source rows 4w .. 4w+3
    const int64_t cc = c0 + c, rr = r0 + 4 * w;
    if (cc >= cols || rr >= rows) continue;
    const int sh = (c & 3) * 8;
    const uint32_t v = ((tile[4 * w][c >> 2] >> sh) & 0xffu) | (((tile[4 * w + 1][c >> 2] >> sh) & 0xffu) << 8) |
                       (((tile[4 * w + 2][c >> 2] >> sh) & 0xffu) << 16) | (((tile[4 * w + 3][c >> 2] >> sh) & 0xffu) << 24);
    *reinterpret_cast<uint32_t*>(dst + cc * rows + rr) = v;
  }
}

// Kernel rows of group g padded from Kg to Kp columns; the padding holds the kernel zero-point (its term vanishes).
__global__ void __launch_bounds__(256) conv_pad_kernel_rows(const int8_t* __restrict__ ker, int64_t rows, int64_t Kg, int64_t Kp,
                                                            int zp_ker, int8_t* __restrict__ w) {
  const int64_t total = rows * Kp, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int64_t r = t / Kp, k = t - r * Kp;
    w[t] = k < Kg ? ker[r * Kg + k] : (int8_t)zp_ker;
  }
}

// The GEMM's result for group g is [N*P, Og] (P = OH*OW).  Channel-first output: out[n, g*Og + j, p] = c[n*P + p, j],
// a 32x32 tile transpose per image; channel-last output with groups: out[m, g*Og + j] = c[m, j].
__global__ void __launch_bounds__(256) conv_scatter_nchw_kernel(const int32_t* __restrict__ c, int64_t P, int64_t Og, int64_t O,
                                                                int g, int32_t* __restrict__ out) {
  __shared__ int32_t tile[32][33];
  const int64_t n = blockIdx.z, p0 = (int64_t)blockIdx.x * 32, j0 = (int64_t)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int64_t pp = p0 + r, j = j0 + tx;
    tile[r][tx] = (pp < P && j < Og) ? c[(n * P + pp) * Og + j] : 0;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int64_t j = j0 + r, pp = p0 + tx;
    if (j < Og && pp < P) out[(n * O + (int64_t)g * Og + j) * P + pp] = tile[tx][r];
  }
}

__global__ void __launch_bounds__(256) conv_scatter_nhwc_kernel(const int32_t* __restrict__ c, int64_t M, int64_t Og, int64_t O,
                                                                int g, int32_t* __restrict__ out) {
  const int64_t total = M * Og, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int64_t m = t / Og, j = t - m * Og;
    out[m * O + (int64_t)g * Og + j] = c[t];
  }
}

unsigned flat_grid(b200q_ctx* ctx, int64_t items) {
  int64_t b = (items + 255) / 256, cap = (int64_t)ctx->sm_count * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

}  // namespace

int launch_quantize_per_group(b200q_ctx* ctx, const float* x, int64_t n, int64_t group_size, int num_bits, int8_t* q,
                              double* scales64, float* scales32) {
  ProfScope prof(ctx, KK_WEIGHTS);
  if (n == 0) return 0;
  const int64_t groups = (n + group_size - 1) / group_size;
  const double bound = (double)((1 << (num_bits - 1)) - 1);
  const float qmin = -(float)(1 << (num_bits - 1)), qmax = (float)((1 << (num_bits - 1)) - 1);
  int64_t blocks = (groups + 7) / 8, cap = (int64_t)ctx->sm_count * 8;
  if (blocks > cap) blocks = cap;
  const bool vec = group_size % 4 == 0 && n % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(q) & 3u) == 0;
  if (vec) group_quantize_kernel<true><<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, n, group_size, groups, bound, qmin, qmax, q, scales64, scales32);
  else group_quantize_kernel<false><<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, n, group_size, groups, bound, qmin, qmax, q, scales64, scales32);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_dequantize_per_group(b200q_ctx* ctx, const int8_t* q, int64_t n, int64_t group_size, const double* scales64, double* y64,
                                float* y32) {
  ProfScope prof(ctx, KK_WEIGHTS);
  if (n == 0) return 0;
  group_dequantize_kernel<<<flat_grid(ctx, n), 256, 0, ctx->stream>>>(q, n, group_size, scales64, y64, y32);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_quantized_conv2d(b200q_ctx* ctx, const int8_t* in, const int8_t* ker, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                            int64_t KH, int64_t KW, int sh, int sw, int pt, int pb, int pl, int pr, int dh, int dw, int groups,
                            int zp_in, int zp_ker, int layout, int32_t* out) {
  ConvGeom p;
  p.N = N; p.C = C; p.H = H; p.W = W; p.O = O; p.KH = KH; p.KW = KW;
  p.sh = sh; p.sw = sw; p.pt = pt; p.pl = pl; p.dh = dh; p.dw = dw;
  p.groups = groups; p.zp_in = zp_in; p.zp_ker = zp_ker; p.layout = layout;
  p.OH = (H + pt + pb - ((KH - 1) * dh + 1)) / sh + 1;   // src/compiler/ir/graph/ops/linalg.ts:236-246
  p.OW = (W + pl + pr - ((KW - 1) * dw + 1)) / sw + 1;
  p.Cg = C / groups; p.Og = O / groups;
  p.Kg = p.Cg * KH * KW;
  p.Kp = (p.Kg + 15) / 16 * 16;
  const int64_t P = p.OH * p.OW, M = N * P;
  if (M == 0 || O == 0) return 0;
  if (p.Kg == 0) {
    B200Q_CHECK_CUDA(cudaMemsetAsync(out, 0, (size_t)M * O * sizeof(int32_t), ctx->stream));
    return 0;
  }
  // With a multiple of 16 channels per group the rows are gathered 16 bytes at a time from a channel-last input; a
  // channel-first input (and its kernel tensor) is re-laid channel-last first, which costs one pass over each.
  const bool out_nchw = layout == 0;
  const bool fast = p.Cg % 16 == 0 && N <= 65535 && O <= 65535 && M < (int64_t(1) << 31) && H * W < (int64_t(1) << 31);
  const bool relay = fast && layout == 0;
  const bool pad_w = p.Kp != p.Kg;                 // never with `fast`
  const bool direct_out = !out_nchw && groups == 1;
  // workspaces: gathered rows (int8); the re-laid input and kernel, or the padded kernel rows of a group (int8);
  // the GEMM's result when it has to be re-laid (channel-first output, or groups)
  const bool aligned = relay || (reinterpret_cast<uintptr_t>(in) & 15u) == 0;   // 16-byte loads of the fast gather
  // A pointwise layer over a channel-last input with one group IS the row matrix: nothing to gather.
  const bool pointwise = fast && aligned && groups == 1 && KH == 1 && KW == 1 && sh == 1 && sw == 1 && pt == 0 && pb == 0 && pl == 0 && pr == 0;
  if (!pointwise && ws_reserve(ctx, ctx->ws_q, (size_t)M * p.Kp)) return 1;
  if (relay && ws_reserve(ctx, ctx->ws_stage_out, (size_t)N * C * H * W)) return 1;
  if ((relay || pad_w) && ws_reserve(ctx, ctx->ws_stage_in, relay ? (size_t)O * p.Kg : (size_t)p.Og * p.Kp)) return 1;
  if (!direct_out && ws_reserve(ctx, ctx->ws_acc, (size_t)M * p.Og * sizeof(int32_t))) return 1;
  int8_t* a = (int8_t*)ctx->ws_q.ptr;
  if (relay) {
    ProfScope prof(ctx, KK_WEIGHTS);
    const int64_t HW = H * W, taps = KH * KW;
    if (HW % 4 == 0 && C % 4 == 0 && (reinterpret_cast<uintptr_t>(in) & 3u) == 0) {
      dim3 gi((unsigned)((HW + 63) / 64), (unsigned)((C + 63) / 64), (unsigned)N);
      conv_relay_i8x4_kernel<<<gi, 256, 0, ctx->stream>>>(in, C, HW, (int8_t*)ctx->ws_stage_out.ptr);
    } else {
      dim3 gi((unsigned)((HW + 31) / 32), (unsigned)((C + 31) / 32), (unsigned)N);
      conv_relay_i8_kernel<<<gi, 256, 0, ctx->stream>>>(in, C, HW, (int8_t*)ctx->ws_stage_out.ptr);
    }
    dim3 gk((unsigned)((taps + 31) / 32), (unsigned)((p.Cg + 31) / 32), (unsigned)O);
    conv_relay_i8_kernel<<<gk, 256, 0, ctx->stream>>>(ker, p.Cg, taps, (int8_t*)ctx->ws_stage_in.ptr);
    ctx->launches += 2;
    B200Q_CHECK_CUDA(cudaGetLastError());
    in = (const int8_t*)ctx->ws_stage_out.ptr;
    ker = (const int8_t*)ctx->ws_stage_in.ptr;
    p.layout = 1;
  }
  for (int g = 0; g < groups; g++) {
    if (pointwise) {
      a = const_cast<int8_t*>(in);
    } else {
      ProfScope prof(ctx, KK_WEIGHTS);
      if (fast && aligned) conv_gather_nhwc16_kernel<<<flat_grid(ctx, M * (p.Cg / 16)), 256, 0, ctx->stream>>>(in, p, g, a);
      else conv_gather_kernel<<<flat_grid(ctx, M * (p.Kp / 16)), 256, 0, ctx->stream>>>(in, p, g, a);
      ctx->launches++;
    }
    const int8_t* w = ker + (int64_t)g * p.Og * p.Kg;
    if (pad_w) {
      ProfScope prof(ctx, KK_WEIGHTS);
      conv_pad_kernel_rows<<<flat_grid(ctx, p.Og * p.Kp), 256, 0, ctx->stream>>>(w, p.Og, p.Kg, p.Kp, zp_ker, (int8_t*)ctx->ws_stage_in.ptr);
      ctx->launches++;
      w = (const int8_t*)ctx->ws_stage_in.ptr;
    }
    B200Q_CHECK_CUDA(cudaGetLastError());
    int32_t* c = direct_out ? out : (int32_t*)ctx->ws_acc.ptr;
    if (int e = gemm_i32_any(ctx, a, w, M, p.Og, p.Kp, zp_in, zp_ker, c)) return e;
    if (!direct_out) {
      ProfScope prof(ctx, KK_WEIGHTS);
      if (out_nchw) {
        dim3 grid((unsigned)((P + 31) / 32), (unsigned)((p.Og + 31) / 32), (unsigned)N);
        conv_scatter_nchw_kernel<<<grid, 256, 0, ctx->stream>>>(c, P, p.Og, O, g, out);
      } else {
        conv_scatter_nhwc_kernel<<<flat_grid(ctx, M * p.Og), 256, 0, ctx->stream>>>(c, M, p.Og, O, g, out);
      }
      ctx->launches++;
      B200Q_CHECK_CUDA(cudaGetLastError());
    }
  }
  return 0;
}

}  // namespace b200q
