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
// |x/s| * 2^-24.  Away from a tie every rounding rule gives the same integer, so
// the fast path rounds with the 1.5*2^23 trick (no conversion instruction) and
// only KEEPS TRACK of whether any element of the thread was unsafe:
//   - closer to a tie than |t| * 2^-21 (a margin of 2.6x over the error above),
//   - outside the clamp range (the fast path does not clamp) or beyond 2^22,
//   - NaN or infinite.
// All of these are folded into two running maxima kept as integers (the bit
// pattern of a non-negative float orders like the float, NaN sorts above all),
// which costs two instructions per element and no branch.  A thread that saw an
// unsafe element (about one element in 10^5 for unit-variance data) recomputes
// its codes with the exact binary64 routines below.
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

struct QuantGuard {
  int tie = 0;  // max of bits(|t - rint(t)| + |t| * 2^-21)
  int mag = 0;  // max of bits(|t|)
  // limit = min(-qmin, qmax) + 0.49: beyond it the unclamped fast code may be wrong
  __device__ __forceinline__ bool unsafe(float limit) const { return tie >= 0x3f000000 || mag > __float_as_int(limit); }
};

// Code of x on the fast path (valid only if the guard stays safe).
__device__ __forceinline__ int quantize_fast(float x, float inv, QuantGuard& g) {
  const float t = __fmul_rn(x, inv);
  const float u = __fadd_rn(t, 12582912.0f);            // 1.5 * 2^23: the sum is rounded to an integer
  const int c = __float_as_int(u) - 0x4B400000;
  const float d = __fsub_rn(t, __fsub_rn(u, 12582912.0f));
  const float e = __fmaf_rn(fabsf(t), 4.76837158203125e-7f, fabsf(d));
  g.tie = max(g.tie, __float_as_int(e));                // NaN has the bit pattern 0x7fffffff
  g.mag = max(g.mag, __float_as_int(fabsf(t)));
  return c;
}

// Four int codes -> one word of four bytes (low byte first).
__device__ __forceinline__ uint32_t pack_codes(int c0, int c1, int c2, int c3) {
  return __byte_perm(__byte_perm((uint32_t)c0, (uint32_t)c1, 0x0040), __byte_perm((uint32_t)c2, (uint32_t)c3, 0x0040), 0x5410);
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
// Small: |acc| < 2^22, converted without a conversion instruction (1.5 * 2^23 trick).
__device__ __forceinline__ float scale_acc_small(int acc, float sv) {
  return __fmul_rn(__fsub_rn(__int_as_float(0x4B400000 + acc), 12582912.0f), sv);
}
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
  // exp(r) = 1 + r + r^2/2 + ... + r^6/720, evaluated in Estrin form: the dependent chain is 4 operations long
  // instead of 6, which matters because the epilogue runs few warps.
  const double r2 = r * r;
  const double a = fma(r, 1.0, 1.0);                        // 1 + r
  const double b = fma(r, 1.0 / 6.0, 0.5);                  // 1/2 + r/6
  const double c = fma(r, 1.0 / 120.0, 1.0 / 24.0);         // 1/24 + r/120
  const double d = fma(r2, 1.0 / 720.0, c);                 // 1/24 + r/120 + r^2/720
  const double hi = fma(r2 * r2, d, 0.0);
  const double p = fma(r2, b, a) + hi;
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

// ---------------------------------------------------------------------------
// Branch-free activations for the fused epilogue.  A thread evaluates 32 of
// them back to back; anything with a call or a data-dependent branch in it
// (the IEEE division, range checks) would stop the compiler from interleaving
// those 32 independent chains.  The sigmoid-based ones are exact (same value as
// sigmoid_ref) for every argument except z < -87 (exp(-z) overflows towards the
// binary32 range limit) and -Inf, where they return an unspecified finite value or
// NaN: callers test `needs_general_act` and redo those elements with apply_act.
// NaN and +Inf arguments give the reference's result without help.
// ---------------------------------------------------------------------------

// Correctly rounded 1/d for finite d in [1, 2^126], branch-free: hardware approximation, one
// Newton step (faithful result), then the better of the result and its neighbour on the side the
// exact residual 1 - d*y points to (the residual of a faithful y is exactly representable).
__device__ __forceinline__ float rcp_rn_ge1(float d) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(d));
  const float e = __fmaf_rn(-d, y, 1.0f);
  y = __fmaf_rn(y, e, y);
  const float r = __fmaf_rn(-d, y, 1.0f);
  const float yc = __int_as_float(__float_as_int(y) + (r > 0.0f ? 1 : -1));
  const float rc = __fmaf_rn(-d, yc, 1.0f);
  return (fabsf(rc) < fabsf(r)) ? yc : y;
}

// sigmoid(z) for z >= -87 (exact), NaN (NaN) and +Inf (1).
__device__ __forceinline__ float sigmoid_fast(float z, const double* tbl) {
  float zc;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(zc) : "f"(z), "f"(100.0f));  // exp(-100) already vanishes against 1; NaN is kept
  const float e = __double2float_rn(exp_f64((double)(-zc), tbl));
  return rcp_rn_ge1(__fadd_rn(1.0f, e));
}

// fround(1.702 * y) with 1.702 a binary64 constant, in binary32 arithmetic: 1.702 = CH + CL + (< 2^-53),
// y*CH is expanded exactly with an FMA.  Differs from the binary64 product only when that product lies
// within 2^-48 (relative) of a rounding boundary, about one argument in 10^7.
__device__ __forceinline__ float mul_1702(float y) {
  const float CH = 1.70200002193450927734375f;             // fl32(1.702)
  const float CL = -2.1934509319976314e-08f;               // fl32(1.702 - CH)
  const float p = __fmul_rn(y, CH);
  const float ep = __fmaf_rn(y, CH, -p);                   // NaN when p overflowed to +-Inf
  const float z = __fadd_rn(p, __fmaf_rn(y, CL, ep));
  return (fabsf(p) == __int_as_float(0x7f800000)) ? p : z;
}

template <int ACT_T>
__device__ __forceinline__ float apply_act_fast(float y, const double* tbl) {
  if (ACT_T == ACT_RELU) return (y > 0.0f) ? y : ((y != y) ? y : 0.0f);
  if (ACT_T == ACT_GELU_SIGMOID) return __fmul_rn(y, sigmoid_fast(mul_1702(y), tbl));
  if (ACT_T == ACT_SILU) return __fmul_rn(y, sigmoid_fast(y, tbl));
  if (ACT_T == ACT_GELU_TANH) {
    // 0.5*(1+tanh(u)) = 1/(1+exp(-2u)), u = sqrt(2/pi)*(y + 0.044715 y^3); binary32, tolerance only
    // (the reference has no tanh form).  Saturates correctly for large |y|.
    const float y2 = y * y;
    const float w = y * fmaf(y2, -0.10294324f, -2.3022082f);   // -2u*log2(e)
    float e, s;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(w));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(s) : "f"(1.0f + e));
    return y * s;
  }
  return y;
}

// Eight sigmoid-based activations at once, written stage by stage: every loop below is one step of the
// computation applied to eight independent elements, so the instruction stream itself is interleaved eight
// ways (the per-element form leaves the compiler with one long dependent chain after another, and with two
// epilogue warps per scheduler nothing else hides those latencies).  Same values as apply_act_fast.
template <int ACT_T>
__device__ __forceinline__ void apply_sigmoid_act_x8(float (&y)[8], const double* tbl) {
  constexpr int W = 8;
  float z[W];
  double x[W], t[W], kd[W], r[W], r2[W], a[W], b[W], c[W], p[W], m[W];
  int k[W];
  float e[W], d[W], g[W], res[W], cand[W], rc[W];
#pragma unroll
  for (int i = 0; i < W; i++) z[i] = (ACT_T == ACT_GELU_SIGMOID) ? mul_1702(y[i]) : y[i];
#pragma unroll
  for (int i = 0; i < W; i++) {
    float zc;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(zc) : "f"(z[i]), "f"(100.0f));
    x[i] = (double)(-zc);
  }
  const double INV = 92.33248261689366, MAGIC = 6755399441055744.0;
  const double HI = __longlong_as_double(0x3F862E42FEE00000LL), LO = __longlong_as_double(0x3D8A39EF35793C76LL);
#pragma unroll
  for (int i = 0; i < W; i++) t[i] = fma(x[i], INV, MAGIC);
#pragma unroll
  for (int i = 0; i < W; i++) { k[i] = __double2loint(t[i]); kd[i] = t[i] - MAGIC; }
#pragma unroll
  for (int i = 0; i < W; i++) r[i] = fma(-kd[i], HI, x[i]);
#pragma unroll
  for (int i = 0; i < W; i++) r[i] = fma(-kd[i], LO, r[i]);
#pragma unroll
  for (int i = 0; i < W; i++) { r2[i] = r[i] * r[i]; a[i] = fma(r[i], 1.0, 1.0); b[i] = fma(r[i], 1.0 / 6.0, 0.5); c[i] = fma(r[i], 1.0 / 120.0, 1.0 / 24.0); }
#pragma unroll
  for (int i = 0; i < W; i++) { c[i] = fma(r2[i], 1.0 / 720.0, c[i]); a[i] = fma(r2[i], b[i], a[i]); b[i] = r2[i] * r2[i]; }
#pragma unroll
  for (int i = 0; i < W; i++) p[i] = a[i] + fma(b[i], c[i], 0.0);
#pragma unroll
  for (int i = 0; i < W; i++) m[i] = tbl[k[i] & 63] * p[i];
#pragma unroll
  for (int i = 0; i < W; i++) e[i] = __double2float_rn(m[i] * __hiloint2double(((k[i] >> 6) + 1023) << 20, 0));
#pragma unroll
  for (int i = 0; i < W; i++) d[i] = __fadd_rn(1.0f, e[i]);
#pragma unroll
  for (int i = 0; i < W; i++) asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(g[i]) : "f"(d[i]));
#pragma unroll
  for (int i = 0; i < W; i++) g[i] = __fmaf_rn(g[i], __fmaf_rn(-d[i], g[i], 1.0f), g[i]);
#pragma unroll
  for (int i = 0; i < W; i++) res[i] = __fmaf_rn(-d[i], g[i], 1.0f);
#pragma unroll
  for (int i = 0; i < W; i++) cand[i] = __int_as_float(__float_as_int(g[i]) + (res[i] > 0.0f ? 1 : -1));
#pragma unroll
  for (int i = 0; i < W; i++) rc[i] = __fmaf_rn(-d[i], cand[i], 1.0f);
#pragma unroll
  for (int i = 0; i < W; i++) y[i] = __fmul_rn(y[i], (fabsf(rc[i]) < fabsf(res[i])) ? cand[i] : g[i]);
}

// True when apply_act_fast<ACT_T>(y) may differ from apply_act(y): compares the bit pattern as an
// unsigned number, which orders the negative floats by magnitude and puts them (and -Inf, -NaN)
// above every positive one.
template <int ACT_T>
__device__ __forceinline__ constexpr unsigned act_general_threshold() {
  return ACT_T == ACT_GELU_SIGMOID ? 0xC24C0000u /* -51.0f: 1.702 * 51 < 87 */
         : ACT_T == ACT_SILU       ? 0xC2AE0000u /* -87.0f */
                                   : 0xFFFFFFFFu;
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

// Out-of-line copy for rarely taken paths (keeps the hot loops small).
static __device__ __noinline__ float apply_act_general(float y, int act, const double* tbl) { return apply_act(y, act, tbl); }

template <int ACT_T>
__device__ __forceinline__ float apply_act_t(float y, const double* tbl) {
  return apply_act(y, ACT_T, tbl);  // the switch folds away: ACT_T is a compile-time constant
}

}  // namespace b200q
