// Device-side arithmetic shared by every kernel of the backend.
//
// The reference's CPU target evaluates f32 expressions as "binary64 operation,
// then one Math.fround" (src/backend/cpu/codegen.ts:172-174,496).  For + - * /
// on two binary32 operands that equals the correctly rounded binary32
// operation (53 >= 2*24+2, so the double rounding is innocuous), so __fmul_rn,
// __fadd_rn and __fdiv_rn reproduce it bit for bit.  The intrinsics (rather
// than * and +) also stop the compiler from contracting a multiply and an add
// into one FMA, which would round once where the reference rounds twice.
// Where an operand is NOT a binary32 value (an int32 accumulator, a binary64
// scale immediate, Math.exp) the functions below go through binary64.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace b200q {

enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU_SIGMOID = 2, ACT_GELU_TANH = 3, ACT_SILU = 4 };

// ---------------------------------------------------------------------------
// Rounding a quotient x / s to the nearest integer, ties toward +infinity.
//
// The streaming kernels evaluate the quotient as t = x * fl32(1/s): two binary32
// roundings, so |t - x/s| <= |x/s| * 2^-23.  Rounding the TRUE quotient to
// binary32 first (the static ops do: fround(x / s)) moves it by at most another
// |x/s| * 2^-24.  An element is therefore safe on the fast path unless the
// fractional part of t lies within |t| * 2^-21 of .5 (a margin of 2.6x); the few
// that do not (about one in 10^5 for unit-variance data) are flagged and redone
// exactly in binary64.  Everything on the fast path is branch-free, so the
// compiler can interleave the independent elements a thread holds; the exact
// path is a separate, rarely taken loop.
// ---------------------------------------------------------------------------

// Math.round for a binary64 value (ties toward +infinity; NaN/Inf pass through:
// for Inf the difference is NaN, the comparison false and floor(Inf) = Inf).
__device__ __forceinline__ double js_round_f64(double t) {
  double r = floor(t);
  return (t - r >= 0.5) ? r + 1.0 : r;
}
__device__ __forceinline__ float js_round_f32(float t) {
  float r = floorf(t);
  return (__fsub_rn(t, r) >= 0.5f) ? r + 1.0f : r;  // t - floor(t) is exact
}

// Fast path shared by both modes.  Returns the int8/uint8 code for x and sets
// `redo` when the element must take the exact path.  NaN gives code 0 (typed-array
// store of NaN) and never asks for a redo.  |t| >= 512 is beyond every 8-bit clamp.
__device__ __forceinline__ int quantize_fast(float x, float inv, float qmin, float qmax, bool& redo) {
  const float t = __fmul_rn(x, inv);
  const float r = floorf(t);
  const float f = __fsub_rn(t, r);                       // exact; NaN when t is +-Inf
  const float at = fabsf(t);
  redo = (fabsf(f - 0.5f) < at * 4.76837158203125e-7f) && (at < 512.0f);
  float q = (f > 0.5f) ? r + 1.0f : r;                   // Inf keeps r = +-Inf
  q = fminf(fmaxf(q, qmin), qmax);
  const int c = (int)q;
  return (x != x) ? 0 : c;
}

// QuantizationParams.quantize (src/compiler/ir/graph/quantization_types.ts:75-79,118-130):
// max(cMin, min(cMax, Math.round(x / s))) in binary64, then an Int8Array store (NaN -> 0).
static __device__ __noinline__ int quantize_exact_p(float x, double s, float qmin, float qmax) {
  if (x != x) return 0;
  float r = (float)js_round_f64((double)x / s);
  return (int)fminf(fmaxf(r, qmin), qmax);
}

// Compiled `quantize` (src/compiler/passes/lowering/quant_math.ts:16-27 as emitted by
// src/backend/cpu/codegen.ts): t = fround(x / s); [t = fround(t + zp);] Math.round; clamp; (v|0).
static __device__ __noinline__ int quantize_exact_c(float x, double s, float zp, float qmin, float qmax) {
  if (x != x) return 0;
  float t = __double2float_rn((double)x / s);
  if (zp != 0.0f) t = __fadd_rn(t, zp);
  float r = js_round_f32(t);
  return (int)fminf(fmaxf(r, qmin), qmax);
}

// fround((double)acc * sv): exact product in binary64 whenever |acc| < 2^24,
// which makes the binary32 multiply identical; otherwise go through binary64.
__device__ __forceinline__ float scale_acc(int acc, float sv) {
  if (abs(acc) < (1 << 24)) return __fmul_rn((float)acc, sv);
  return __double2float_rn((double)acc * (double)sv);
}
// The two halves of scale_acc for callers that pick one per group of elements.
__device__ __forceinline__ float scale_acc_small(int acc, float sv) { return __fmul_rn((float)acc, sv); }
__device__ __forceinline__ float scale_acc_wide(int acc, float sv) { return __double2float_rn((double)acc * (double)sv); }

// ---------------------------------------------------------------------------
// exp for a binary32 argument, evaluated in binary64 (error < 2 ulp of
// binary64) and rounded once to binary32 == Math.fround(Math.exp(x)) except
// when the binary64 value lies within ~2^-52 of a binary32 rounding boundary
// (probability about 1e-8 per evaluation).
//   x = k*ln2/64 + r,  exp(x) = 2^(k>>6) * 2^((k&63)/64) * exp(r),  |r| <= ln2/128
// `tbl` holds 2^(j/64), j = 0..63 (shared memory; see fill_exp2_table).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void fill_exp2_table(double* tbl, int tid, int nthreads) {
  for (int j = tid; j < 64; j += nthreads) tbl[j] = exp2((double)j * (1.0 / 64.0));
}

__device__ __forceinline__ double exp_f64(double xd, const double* tbl) {
  const double INV = 92.33248261689366;               // 64 / ln 2
  const double MAGIC = 6755399441055744.0;            // 1.5 * 2^52: adding it rounds to an integer
  // ln2/64 = HI + LO; HI keeps 32 significant bits so that kd * HI is exact for |kd| < 2^21.
  const double HI = __longlong_as_double(0x3F862E42FEE00000LL);
  const double LO = __longlong_as_double(0x3D8A39EF35793C76LL);
  double t = fma(xd, INV, MAGIC);
  int k = __double2loint(t);
  double kd = t - MAGIC;
  double r = fma(-kd, HI, xd);
  r = fma(-kd, LO, r);
  double p = 1.0 / 720.0;
  p = fma(p, r, 1.0 / 120.0);
  p = fma(p, r, 1.0 / 24.0);
  p = fma(p, r, 1.0 / 6.0);
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  p = fma(p, r, 1.0);
  double m = tbl[k & 63] * p;
  int e = k >> 6;                                      // |e| < 256: 2^e is a normal binary64
  return m * __hiloint2double((e + 1023) << 20, 0);
}

// Branch-free: the argument is clamped to [-160, 128] (exp(128) rounds to +Inf in
// binary32, exp(-160) to 0), NaN is restored by a select.
__device__ __forceinline__ float exp_fround(float x, const double* tbl) {
  const float xc = fminf(fmaxf(x, -160.0f), 128.0f);
  const float r = __double2float_rn(exp_f64((double)xc, tbl));
  return (x != x) ? x : r;
}

// sigmoid as the reference decomposes it (src/compiler/passes/decompose/
// decomposition_pass.ts:197-203): 1 / (1 + exp(-z)), one rounding per op.
__device__ __forceinline__ float sigmoid_ref(float z, const double* tbl) {
  float e = exp_fround(-z, tbl);
  float d = __fadd_rn(1.0f, e);
  return __fdiv_rn(1.0f, d);
}

// Bias add has happened; `y` is the pre-activation value.
template <int ACT_T>
__device__ __forceinline__ float apply_act_t(float y, const double* tbl);

__device__ __forceinline__ float apply_act(float y, int act, const double* tbl) {
  switch (act) {
    case ACT_RELU:  // Math.max(y, 0): NaN stays NaN, -0 becomes +0
      return (y > 0.0f) ? y : ((y != y) ? y : 0.0f);
    case ACT_GELU_SIGMOID: {  // y * sigmoid(fround(1.702 * y)); 1.702 is a binary64 immediate
      float z = __double2float_rn(1.702 * (double)y);
      return __fmul_rn(y, sigmoid_ref(z, tbl));
    }
    case ACT_SILU:
      return __fmul_rn(y, sigmoid_ref(y, tbl));
    case ACT_GELU_TANH: {
      // The reference has no tanh form; binary32 arithmetic, checked to tolerance only.
      float y3 = __fmul_rn(__fmul_rn(y, y), y);
      float in = __fadd_rn(y, __fmul_rn(0.044715f, y3));
      float u = __fmul_rn(0.7978845608028654f, in);
      float au = fabsf(u);
      float e2 = __expf(-2.0f * au);                       // in (0, 1]
      float th = __fdividef(1.0f - e2, 1.0f + e2);
      th = copysignf(th, u);
      return __fmul_rn(__fmul_rn(0.5f, y), __fadd_rn(1.0f, th));
    }
    default:
      return y;
  }
}

template <int ACT_T>
__device__ __forceinline__ float apply_act_t(float y, const double* tbl) {
  return apply_act(y, ACT_T, tbl);  // the switch folds away: ACT_T is a compile-time constant
}

}  // namespace b200q
