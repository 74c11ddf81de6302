// int8 x int8 -> int32 contraction on the CUDA cores (dp4a) and the unfused
// per-channel tail.  This is the correctness anchor of the backend on the
// device: it handles every shape, stride and zero-point, and the tensor-core
// kernel is checked against it at sizes the CPU oracle cannot finish.
//
// Reference: quantized_dot lowering, src/compiler/passes/lowering/rules/
// quantization.ts:23-42 (C[m,n] = sum_k (A-zpA)*(B-zpB), int32); tail,
// src/compiler/passes/quantization/quantization_pass.ts:427-456.
#include "common.cuh"
#include "kernels.cuh"
#include "quant_math.cuh"

namespace b200q {

namespace {

constexpr int TM = 64, TN = 64, TK = 64;  // block tile; 256 threads, 4x4 outputs each

// A is [M,K] row-major, W is [N,K] row-major (K contiguous in both).
template <bool ZP>
__global__ void __launch_bounds__(256) gemm_i8_simt_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ W, int64_t M,
                                                           int64_t N, int64_t K, int zpA, int zpB, int32_t* __restrict__ C) {
  __shared__ __align__(16) int8_t sA[TM][TK + 16];
  __shared__ __align__(16) int8_t sW[TN][TK + 16];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * TM, n0 = (int64_t)blockIdx.x * TN;
  int acc[4][4] = {};
  for (int64_t k0 = 0; k0 < K; k0 += TK) {
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      int r = i / TK, c = i % TK;
      int64_t m = m0 + r, k = k0 + c;
      // Padding must not contribute: with zero-points the padded operand equals its zero-point.
      sA[r][c] = (m < M && k < K) ? A[m * K + k] : (int8_t)(ZP ? zpA : 0);
      int64_t n = n0 + r;
      sW[r][c] = (n < N && k < K) ? W[n * K + k] : (int8_t)(ZP ? zpB : 0);
    }
    __syncthreads();
    if (!ZP) {
#pragma unroll 4
      for (int kk = 0; kk < TK; kk += 4) {
        int a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; i++) a[i] = *reinterpret_cast<const int*>(&sA[ty * 4 + i][kk]);
#pragma unroll
        for (int j = 0; j < 4; j++) b[j] = *reinterpret_cast<const int*>(&sW[tx * 4 + j][kk]);
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++) acc[i][j] = __dp4a(a[i], b[j], acc[i][j]);
      }
    } else {
      for (int kk = 0; kk < TK; kk++) {
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
          for (int j = 0; j < 4; j++)
            acc[i][j] += ((int)sA[ty * 4 + i][kk] - zpA) * ((int)sW[tx * 4 + j][kk] - zpB);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int64_t m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int64_t n = n0 + tx * 4 + j;
      if (n < N) C[m * N + n] = acc[i][j];
    }
  }
}

// out[m,n] = act( fround( fround(acc * fround(aScale[m]*wScale[n])) + bias[n] ) ), or its
// static requantization.  One thread per 4 consecutive columns when N % 4 == 0.
__global__ void __launch_bounds__(256) epilogue_kernel(const int32_t* __restrict__ acc, int64_t M, int64_t N,
                                                       const float* __restrict__ a_scales, const float* __restrict__ w_scales,
                                                       const float* __restrict__ bias, int act, float* __restrict__ out_f32,
                                                       int8_t* __restrict__ out_q, double q_scale, float q_inv, int q_exact,
                                                       double tensor_scale) {
  __shared__ double tbl[EXP2_TABLE_SIZE];
  fill_exp2_table(tbl, threadIdx.x, blockDim.x);
  __syncthreads();
  const int64_t total = M * N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t m = i / N, n = i - m * N;
    float y;
    if (w_scales != nullptr) {
      float sv = a_scales ? __fmul_rn(a_scales[m], w_scales[n]) : w_scales[n];
      y = scale_acc(acc[i], sv);
    } else {
      // the compiled `dequantize` of a per-tensor scale (quant_math.ts:29-34): the scale is a binary64 immediate
      y = __double2float_rn((double)acc[i] * tensor_scale);
    }
    if (bias) y = __fadd_rn(y, bias[n]);
    y = apply_act(y, act, tbl);
    if (out_f32) out_f32[i] = y;
    if (out_q) {
      QuantGuard guard;
      int c = quantize_fast(y, q_inv, guard);
      if (q_exact || guard.unsafe(127.49f)) c = quantize_exact_c(y, q_scale, 0.0f, -128.0f, 127.0f);
      out_q[i] = (int8_t)c;
    }
  }
}

// Zero-points on the tensor cores: sum_k (a - za)(w - zw) = sum_k a w - zw * sum_k a - za * sum_k w + K za zw, all in
// 32-bit two's-complement arithmetic like the accumulator itself.  Row sums of an int8 matrix, one warp per row:
__global__ void __launch_bounds__(256) row_sum_i8_kernel(const int8_t* __restrict__ a, int64_t rows, int64_t K, int32_t* __restrict__ sums) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const bool vec = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15u) == 0);
  for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const int8_t* row = a + r * K;
    int s = 0;
    if (vec) {
      for (int64_t k = 16 * lane; k < K; k += 512) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + k));
        s = __dp4a((int)v.x, 0x01010101, s);
        s = __dp4a((int)v.y, 0x01010101, s);
        s = __dp4a((int)v.z, 0x01010101, s);
        s = __dp4a((int)v.w, 0x01010101, s);
      }
    } else {
      for (int64_t k = lane; k < K; k += 32) s += row[k];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) sums[r] = s;
  }
}

// c[m,n] += K za zw - zw * row_a[m] - za * row_w[n]  (unsigned arithmetic: wraps like the reference's ToInt32 sum)
__global__ void __launch_bounds__(256) zero_point_fix_kernel(int32_t* __restrict__ c, int64_t M, int64_t N, const int32_t* __restrict__ row_a,
                                                             const int32_t* __restrict__ row_w, int za, int zw, uint32_t kzz) {
  const int64_t total = M * N, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t m = i / N, n = i - m * N;
    c[i] = (int32_t)((uint32_t)c[i] + kzz - (uint32_t)zw * (uint32_t)row_a[m] - (uint32_t)za * (uint32_t)row_w[n]);
  }
}

// ui8 codes as int8 codes 128 lower (one bit flipped): u - zp == (u - 128) - (zp - 128), so an unsigned operand of a
// contraction is the signed one with its zero-point moved by 128.
__global__ void __launch_bounds__(256) shift_u8_i8_kernel(const uint8_t* __restrict__ src, int64_t n, int8_t* __restrict__ dst) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x, tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
  const int64_t n16 = vec ? n / 16 : 0;
  for (int64_t i = tid; i < n16; i += stride) {
    uint4 v = __ldcs(reinterpret_cast<const uint4*>(src) + i);
    v.x ^= 0x80808080u; v.y ^= 0x80808080u; v.z ^= 0x80808080u; v.w ^= 0x80808080u;
    reinterpret_cast<uint4*>(dst)[i] = v;
  }
  for (int64_t i = n16 * 16 + tid; i < n; i += stride) dst[i] = (int8_t)(src[i] ^ 0x80u);
}

}  // namespace

int launch_shift_u8_i8(b200q_ctx* ctx, const uint8_t* src, int64_t n, int8_t* dst) {
  ProfScope prof(ctx, KK_QUANT_STATIC);
  if (n == 0) return 0;
  int64_t blocks = (n / 16 + 255) / 256 + 1;
  if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
  shift_u8_i8_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(src, n, dst);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// `sums` receives M + N words (row sums of A, then of W); c is corrected in place.
int launch_zero_point_fix(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K, int zpA, int zpB,
                          int32_t* sums, int32_t* C) {
  ProfScope prof(ctx, KK_GEMM_SIMT);
  if (M == 0 || N == 0) return 0;
  const unsigned cap = (unsigned)ctx->sm_count * 8;
  const int64_t ba = (M + 7) / 8, bw = (N + 7) / 8;
  row_sum_i8_kernel<<<(unsigned)(ba < cap ? ba : cap), 256, 0, ctx->stream>>>(A, M, K, sums);
  row_sum_i8_kernel<<<(unsigned)(bw < cap ? bw : cap), 256, 0, ctx->stream>>>(W_nk, N, K, sums + M);
  int64_t blocks = (M * N + 255) / 256;
  if (blocks > (int64_t)ctx->sm_count * 16) blocks = (int64_t)ctx->sm_count * 16;
  const uint32_t kzz = (uint32_t)K * (uint32_t)zpA * (uint32_t)zpB;
  zero_point_fix_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(C, M, N, sums, sums + M, zpA, zpB, kzz);
  ctx->launches += 3;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_gemm_i8_simt(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K, int zpA, int zpB,
                        int32_t* C) {
  ProfScope prof(ctx, KK_GEMM_SIMT);
  if (M == 0 || N == 0) return 0;
  dim3 grid((unsigned)((N + TN - 1) / TN), (unsigned)((M + TM - 1) / TM));
  B200Q_REQUIRE(grid.y <= 65535, "int8 gemm (simt): M too large for one launch (%lld rows)", (long long)M);
  if (zpA == 0 && zpB == 0)
    gemm_i8_simt_kernel<false><<<grid, 256, 0, ctx->stream>>>(A, W_nk, M, N, K, 0, 0, C);
  else
    gemm_i8_simt_kernel<true><<<grid, 256, 0, ctx->stream>>>(A, W_nk, M, N, K, zpA, zpB, C);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

int launch_epilogue(b200q_ctx* ctx, const int32_t* acc, int64_t M, int64_t N, const float* a_scales, const float* w_scales,
                    const float* bias, int act, float* out_f32, int8_t* out_q, double q_scale, double tensor_scale) {
  ProfScope prof(ctx, KK_EPILOGUE);
  if (M == 0 || N == 0) return 0;
  float q_inv = 0.0f;
  int q_exact = 0;
  if (out_q) {
    q_inv = (float)(1.0 / q_scale);
    float a = q_inv < 0 ? -q_inv : q_inv;
    q_exact = !(a >= 1.17549435e-38f && a <= 3.402823466e38f);
  }
  int64_t blocks = (M * N + 255) / 256;
  int64_t cap = (int64_t)ctx->sm_count * 16;
  if (blocks > cap) blocks = cap;
  epilogue_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(acc, M, N, a_scales, w_scales, bias, act, out_f32, out_q, q_scale,
                                                            q_inv, q_exact, tensor_scale);
  ctx->launches++;
  B200Q_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace b200q
