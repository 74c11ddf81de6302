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

enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU_SIGMOID = 2, ACT_GELU_TANH = 3, ACT_SILU = 4,
                 // internal: the sigmoid forms through the hardware exponential and reciprocal (tolerance only)
                 ACT_GELU_SIGMOID_APPROX = 5, ACT_SILU_APPROX = 6,
                 ACT_GELU_SIGMOID_F32 = 7, ACT_SILU_F32 = 8 };

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

// Order-preserving keys of a row's range, for atomicMax on plain 32-bit words that start at zero.
// range_key_max(v) grows with v, range_key_min(v) grows as v falls; both are at least 1 for every non-NaN v (NaN is
// never published), so 0 means "nothing seen", which decodes to -Inf (maximum) / +Inf (minimum): the values an
// empty or all-NaN row has before the scale rule replaces them (quantization_types.ts:308-316).
__device__ __forceinline__ uint32_t range_key_max(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t range_key_min(float v) { return ~range_key_max(v); }
__device__ __forceinline__ float range_max_from_key(uint32_t k) {
  if (k == 0u) return __int_as_float(0xff800000);
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ float range_min_from_key(uint32_t k) {
  if (k == 0u) return __int_as_float(0x7f800000);
  return range_max_from_key(~k);
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
// Packed binary32 arithmetic of sm_100: one instruction works on a pair of floats held in a 64-bit register
// (round to nearest even per element, no flush to zero: the same values as the scalar instructions).
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_sub(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_dup(float a) { return f2_pack(a, a); }

// Leanest form of the fast code, for finite elements of an ordinary per-token row: the four codes, and the running
// maximum of |t - rint t| (how close any element came to a tie).  t = x * inv, u = t + 1.5*2^23 (the rounding), and
// the code is the low byte of u's bit pattern (|t| <= 127.00002 here, so no clamp; 0x4B400000 + code keeps the code's
// two's complement in its low byte).  Packed arithmetic: eight floating-point instructions per four elements.
// `inv2` and `magic2` hold the reciprocal scale and 1.5*2^23 in both halves.
__device__ __forceinline__ uint32_t pack4_fast_lean(const float4& v, uint64_t inv2, uint64_t magic2, float& far) {
  const uint64_t t01 = f2_mul(f2_pack(v.x, v.y), inv2), t23 = f2_mul(f2_pack(v.z, v.w), inv2);
  const uint64_t u01 = f2_add(t01, magic2), u23 = f2_add(t23, magic2);
  const uint64_t d01 = f2_sub(t01, f2_sub(u01, magic2)), d23 = f2_sub(t23, f2_sub(u23, magic2));
  float d0, d1, d2, d3, u0, u1, u2, u3;
  f2_unpack(d01, d0, d1);
  f2_unpack(d23, d2, d3);
  f2_unpack(u01, u0, u1);
  f2_unpack(u23, u2, u3);
  far = fmaxf(fmaxf(fmaxf(far, fabsf(d0)), fmaxf(fabsf(d1), fabsf(d2))), fabsf(d3));
  const uint32_t lo = __byte_perm(__float_as_uint(u0), __float_as_uint(u1), 0x0040);   // bytes: u0.b0, u1.b0
  const uint32_t hi = __byte_perm(__float_as_uint(u2), __float_as_uint(u3), 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

// The same four codes when the row may hold values the range pass has not seen as such (NaN, +-Inf: the range came
// from elsewhere): `far` is kept with NaN-PROPAGATING three-input maxima (d is NaN for a NaN or infinite element), so
// the caller's test must be !(far < threshold).
__device__ __forceinline__ uint32_t pack4_fast_lean_nan(const float4& v, uint64_t inv2, uint64_t magic2, float& far) {
  const uint64_t t01 = f2_mul(f2_pack(v.x, v.y), inv2), t23 = f2_mul(f2_pack(v.z, v.w), inv2);
  const uint64_t u01 = f2_add(t01, magic2), u23 = f2_add(t23, magic2);
  const uint64_t d01 = f2_sub(t01, f2_sub(u01, magic2)), d23 = f2_sub(t23, f2_sub(u23, magic2));
  float d0, d1, d2, d3, u0, u1, u2, u3;
  f2_unpack(d01, d0, d1);
  f2_unpack(d23, d2, d3);
  f2_unpack(u01, u0, u1);
  f2_unpack(u23, u2, u3);
  asm("max.NaN.f32 %0, %0, %1, %2;" : "+f"(far) : "f"(fabsf(d0)), "f"(fabsf(d1)));
  asm("max.NaN.f32 %0, %0, %1, %2;" : "+f"(far) : "f"(fabsf(d2)), "f"(fabsf(d3)));
  const uint32_t lo = __byte_perm(__float_as_uint(u0), __float_as_uint(u1), 0x0040);
  const uint32_t hi = __byte_perm(__float_as_uint(u2), __float_as_uint(u3), 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

// tie tracking only: in a per-token row |x * (127/absmax)| <= 127 (1 + 2^-23) by construction, so the magnitude
// needs no watching; a NaN element still trips the guard through `e`.
__device__ __forceinline__ int quantize_fast_bounded(float x, float inv, int& tie) {
  const float t = __fmul_rn(x, inv);
  const float u = __fadd_rn(t, 12582912.0f);
  const int c = __float_as_int(u) - 0x4B400000;
  const float d = __fsub_rn(t, __fsub_rn(u, 12582912.0f));
  const float e = __fmaf_rn(fabsf(t), 4.76837158203125e-7f, fabsf(d));
  tie = max(tie, __float_as_int(e));
  return c;
}

// ---------------------------------------------------------------------------
// exp for a binary32 argument, evaluated in binary64 (error about 1.2 ulp of
// binary64) and rounded once to binary32 == Math.fround(Math.exp(x)) except
// when the binary64 value lies within ~2^-52 of a binary32 rounding boundary
// (probability of the order of 1e-9 per evaluation).
//   x = k*ln2/256 + r,  exp(x) = 2^(k>>8) * 2^((k&255)/256) * exp(r),  |r| <= ln2/512 (1 + 2^-7)
// Few binary64 operations on purpose (eight): they issue at a fraction of the binary32 rate.
//  * k comes from a binary32 multiply-add (1.5*2^23 trick); it may be the second nearest integer when
//    x*256/ln2 is within 0.002 of a half, which only widens |r| by that much;
//  * k becomes a binary64 number through the bit pattern of 2^52 + 2^31 + k (exact);
//  * exp(r) - 1 = r + r^2 (1/2 + r/6 + r^2/24) (truncation error < 4e-17), folded into the table
//    product with one FMA: T + T*q;
//  * 2^(k>>8) is added to the exponent field (the product is in [0.99, 2.01), |k>>8| < 160).
// `tbl` holds 2^(j/256), j = 0..255, correctly rounded (shared memory; see fill_exp2_table).
// ---------------------------------------------------------------------------
constexpr int EXP2_TABLE_SIZE = 256;
static __device__ const unsigned long long kExp2TableBits[EXP2_TABLE_SIZE] = {
#include "exp2_table.inc"
};

__device__ __forceinline__ void fill_exp2_table(double* tbl, int tid, int nthreads) {
  for (int j = tid; j < EXP2_TABLE_SIZE; j += nthreads) tbl[j] = __longlong_as_double((long long)kExp2TableBits[j]);
}

constexpr float EXP_INV_F = 369.329930467574632f;               // 256 / ln 2
constexpr float EXP_MAGIC_F = 12582912.0f;                      // 1.5 * 2^23
constexpr int EXP_MAGIC_BITS = 0x4B400000;
constexpr double EXP_MAGIC_D = 4503601774854144.0;              // 2^52 + 2^31
// ln2/256 = HI + LO; HI keeps 32 significant bits so that k * HI is exact for |k| < 2^21.
#define B200Q_EXP_HI __longlong_as_double(0x3F662E42FEE00000LL)
#define B200Q_EXP_LO __longlong_as_double(0x3D6A39EF35793C76LL)

// exp(x) rounded to binary32 for x in [-160, 128] (any other finite x or NaN gives an unspecified value, no trap).
__device__ __forceinline__ float exp_core(float x, const double* tbl) {
  const float tf = __fmaf_rn(x, EXP_INV_F, EXP_MAGIC_F);
  const int k = __float_as_int(tf) - EXP_MAGIC_BITS;
  const double xd = (double)x;
  const double kd = __hiloint2double(0x43300000, k ^ (int)0x80000000) - EXP_MAGIC_D;
  double r = fma(-kd, B200Q_EXP_HI, xd);
  r = fma(-kd, B200Q_EXP_LO, r);
  const double r2 = r * r;
  double b = fma(r, 1.0 / 6.0, 0.5);
  b = fma(r2, 1.0 / 24.0, b);
  const double q = fma(r2, b, r);
  const double t = tbl[k & (EXP2_TABLE_SIZE - 1)];
  const double m = fma(t, q, t);
  const int hi = __double2hiint(m) + ((k >> 8) << 20);
  return __double2float_rn(__hiloint2double(hi, __double2loint(m)));
}

// Branch-free: the argument is clamped to [-160, 128] (exp(128) rounds to +Inf in
// binary32, exp(-160) to 0), NaN is restored by a select.
__device__ __forceinline__ float exp_fround(float x, const double* tbl) {
  const float xc = fminf(fmaxf(x, -160.0f), 128.0f);
  const float r = exp_core(xc, tbl);
  return (x != x) ? x : r;
}

// ---------------------------------------------------------------------------
// Branch-free activations for the fused epilogue.  A thread evaluates 32 of
// them back to back; anything with a call or a data-dependent branch in it
// (the IEEE division, range checks) would stop the compiler from interleaving
// those 32 independent chains.  The sigmoid-based ones give the same value as
// sigmoid_ref for EVERY argument: large negative arguments (exp(-z) near or
// beyond the binary32 range, where 1/(1+e) is subnormal or zero), +-Inf and NaN
// go through the same instructions as ordinary ones.
// ---------------------------------------------------------------------------

// Correctly rounded 1/d for d in [1, +Inf], branch-free.  The hardware approximation and one Newton step
// run on d * 2^-32 (so that neither d up to 2^128 nor its reciprocal leaves the normal range) and give a
// faithful value; scaling back by 2^-32 is exact for a normal result and rounds onto the subnormal grid
// otherwise, still within one grid step of 1/d.  The answer is then the better of that value and its
// neighbour on the side the residual 1 - d*y points to (residuals come from one FMA, subnormal operands
// included).  d = +Inf gives 0 by a final select.
__device__ __forceinline__ float rcp_rn_ge1(float d) {
  const float ds = __fmul_rn(d, 2.3283064365386963e-10f);   // 2^-32
  float g;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(g) : "f"(ds));
  g = __fmaf_rn(g, __fmaf_rn(-ds, g, 1.0f), g);
  const float y = __fmul_rn(g, 2.3283064365386963e-10f);
  const float r = __fmaf_rn(-d, y, 1.0f);
  const float yc = __int_as_float(__float_as_int(y) + (r > 0.0f ? 1 : -1));
  const float rc = __fmaf_rn(-d, yc, 1.0f);
  const float best = (fabsf(rc) < fabsf(r)) ? yc : y;
  return (d == __int_as_float(0x7f800000)) ? 0.0f : best;
}

// sigmoid(z) = 1 / (1 + exp(-z)) with one rounding per operation, any z.  -z is clamped to [-100, 128]:
// exp(-100) already vanishes against 1, exp(128) is +Inf like exp of anything larger; a NaN argument
// becomes -100 here and is restored by the caller's final product with the NaN pre-activation.
__device__ __forceinline__ float sigmoid_fast(float z, const double* tbl) {
  const float xc = fminf(fmaxf(-z, -100.0f), 128.0f);
  return rcp_rn_ge1(__fadd_rn(1.0f, exp_core(xc, tbl)));
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
  if (ACT_T == ACT_GELU_SIGMOID_APPROX || ACT_T == ACT_SILU_APPROX) {
    // x * sigmoid(z) with sigmoid(z) = 1 / (1 + 2^(-z log2 e)): relative error about 2^-21, saturates correctly
    // (2^+big = Inf -> 1/Inf = 0; 2^-big = 0 -> 1), NaN stays NaN.
    const float z = (ACT_T == ACT_GELU_SIGMOID_APPROX) ? 1.702f * y : y;
    float e, sg;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(sg) : "f"(1.0f + e));
    return y * sg;
  }
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
  float z[W], xf[W];
  double x[W], kd[W], r[W], r2[W], b[W], q[W], m[W];
  int k[W];
  float e[W], d[W], ds[W], g[W], res[W], cand[W], rc[W];
#pragma unroll
  for (int i = 0; i < W; i++) z[i] = (ACT_T == ACT_GELU_SIGMOID) ? mul_1702(y[i]) : y[i];
#pragma unroll
  for (int i = 0; i < W; i++) xf[i] = fminf(fmaxf(-z[i], -100.0f), 128.0f);
#pragma unroll
  for (int i = 0; i < W; i++) k[i] = __float_as_int(__fmaf_rn(xf[i], EXP_INV_F, EXP_MAGIC_F)) - EXP_MAGIC_BITS;
#pragma unroll
  for (int i = 0; i < W; i++) { x[i] = (double)xf[i]; kd[i] = __hiloint2double(0x43300000, k[i] ^ (int)0x80000000) - EXP_MAGIC_D; }
#pragma unroll
  for (int i = 0; i < W; i++) r[i] = fma(-kd[i], B200Q_EXP_HI, x[i]);
#pragma unroll
  for (int i = 0; i < W; i++) r[i] = fma(-kd[i], B200Q_EXP_LO, r[i]);
#pragma unroll
  for (int i = 0; i < W; i++) { r2[i] = r[i] * r[i]; b[i] = fma(r[i], 1.0 / 6.0, 0.5); }
#pragma unroll
  for (int i = 0; i < W; i++) b[i] = fma(r2[i], 1.0 / 24.0, b[i]);
#pragma unroll
  for (int i = 0; i < W; i++) { q[i] = fma(r2[i], b[i], r[i]); m[i] = tbl[k[i] & (EXP2_TABLE_SIZE - 1)]; }
#pragma unroll
  for (int i = 0; i < W; i++) m[i] = fma(m[i], q[i], m[i]);
#pragma unroll
  for (int i = 0; i < W; i++)
    e[i] = __double2float_rn(__hiloint2double(__double2hiint(m[i]) + ((k[i] >> 8) << 20), __double2loint(m[i])));
#pragma unroll
  for (int i = 0; i < W; i++) { d[i] = __fadd_rn(1.0f, e[i]); ds[i] = __fmul_rn(d[i], 2.3283064365386963e-10f); }
#pragma unroll
  for (int i = 0; i < W; i++) asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(g[i]) : "f"(ds[i]));
#pragma unroll
  for (int i = 0; i < W; i++) g[i] = __fmaf_rn(g[i], __fmaf_rn(-ds[i], g[i], 1.0f), g[i]);
#pragma unroll
  for (int i = 0; i < W; i++) g[i] = __fmul_rn(g[i], 2.3283064365386963e-10f);
#pragma unroll
  for (int i = 0; i < W; i++) res[i] = __fmaf_rn(-d[i], g[i], 1.0f);
#pragma unroll
  for (int i = 0; i < W; i++) cand[i] = __int_as_float(__float_as_int(g[i]) + (res[i] > 0.0f ? 1 : -1));
#pragma unroll
  for (int i = 0; i < W; i++) rc[i] = __fmaf_rn(-d[i], cand[i], 1.0f);
#pragma unroll
  for (int i = 0; i < W; i++) {
    const float best = (fabsf(rc[i]) < fabsf(res[i])) ? cand[i] : g[i];
    y[i] = __fmul_rn(y[i], (d[i] == __int_as_float(0x7f800000)) ? 0.0f : best);
  }
}

// ---------------------------------------------------------------------------
// exp in binary32 arithmetic only, for the sigmoid tails of the tensor-core kernel (binary64 instructions share
// a pipe with the tensor cores and cost several times their usual price while MMAs are in flight).
//   x in [-18, 88.75]:  k = rint(256 x),  c = x - k/256 (exact: the grid is a power of two, |c| <= 2^-9),
//   exp(x) = E1[k >> 8] * E2[k & 255] * exp(c),  E1[a] = exp(a), E2[b] = exp(b/256) held as hi + lo pairs,
//   exp(c) = 1 + c + c^2 (1/2 + c/6 + c^2/24)  (truncation < 2^-52; the bracket times c^2 is below 2^-19).
// The product is carried as h + low with |low| << ulp(h) and an error below 2^-40 h (not one wrong rounding in
// 1.9e8 random arguments at that margin); the result RN(h + low) is CERTIFIED when h + (low +- 2^-38 h) round to the
// same binary32 number, which fails for about one argument in 11000 -- those are redone in binary64 by the caller.
// Arguments of 88.7228394 and more give +Inf like fround(Math.exp(x)); below -18, exp(x) < 2^-25 and 1 + exp(x)
// rounds to 1 whatever its bits, so the clamp is invisible to a sigmoid.
// ---------------------------------------------------------------------------
constexpr float EXP_OVERFLOW_F = 88.72283935546875f;   // the smallest binary32 x whose exp rounds to +Inf
constexpr int EXP_FF_A_MIN = -18, EXP_FF_A_COUNT = 107, EXP_FF_ENTRIES = EXP_FF_A_COUNT + 256;
struct ExpPair { unsigned hi, lo; };
static __device__ const ExpPair kExpFfTable[EXP_FF_ENTRIES] = {
#include "exp_ff_table.inc"
};
// Shared-memory copy: hi words of all entries, then lo words (4-byte loads spread over the banks, and two
// elements' words land in a register pair without shuffling).
__device__ __forceinline__ void fill_exp_ff_table(float* tbl, int tid, int nthreads) {
  for (int j = tid; j < EXP_FF_ENTRIES; j += nthreads) {
    tbl[j] = __uint_as_float(kExpFfTable[j].hi);
    tbl[EXP_FF_ENTRIES + j] = __uint_as_float(kExpFfTable[j].lo);
  }
}

// Eight sigmoid-based activations at once, written stage by stage over four PAIRS of elements: every loop below is
// one step of the computation in packed binary32 arithmetic (two lanes per instruction, each lane rounded like the
// scalar instruction), so the instruction stream is interleaved four ways and half as long as the scalar form (with two
// epilogue warps per scheduler nothing else hides those latencies).  Same values as apply_act (bit for bit).
// Negated quantities are formed by multiplying with a negated factor (exact), since the packed forms take no sign
// modifiers.  `tbl`: the table of fill_exp_ff_table in shared memory.  Warp-collective (one vote).
template <int ACT_T, int W>
__device__ __forceinline__ void apply_sigmoid_act_wide(float (&y)[W], const float* tbl) {
  static_assert(W % 2 == 0, "elements are processed in pairs");
  constexpr int H = W / 2;
  const uint64_t MAG2 = f2_dup(12582912.0f), ONE2 = f2_dup(1.0f);
  float xf[W], ea[W], eb[W], g[W], res[W], rc[W], cand[W], sg[W];
  uint64_t c2[H], h2[H], low2[H], nd2[H], nds2[H], g2[H];
  int k[W];
  {
    uint64_t nz2[H];
    if (ACT_T == ACT_GELU_SIGMOID) {
      // -z = -(1.702 y) with 1.702 held as CH + CL; |y| is clamped first (1e30 saturates the sigmoid either way) so that
      // no product overflows.  A NaN leaves the clamp as -1e30; the final product with y restores it.
      const uint64_t CH2 = f2_dup(1.70200002193450927734375f), NCH2 = f2_dup(-1.70200002193450927734375f),
                     NCL2 = f2_dup(2.1934509319976314e-08f), ZERO2 = f2_dup(0.0f);
#pragma unroll
      for (int i = 0; i < H; i++) {
        // The negated product comes out of an fma with a zero addend, not a mul: a packed mul feeding a packed add was
        // seen to be merged into one fused operation here (one rounding fewer), whatever the .rn on both.
        const uint64_t yc = f2_pack(fminf(fmaxf(y[2 * i], -1e30f), 1e30f), fminf(fmaxf(y[2 * i + 1], -1e30f), 1e30f));
        const uint64_t pp = f2_mul(yc, CH2), pn = f2_fma(yc, NCH2, ZERO2);
        nz2[i] = f2_add(pn, f2_fma(yc, NCL2, f2_fma(yc, NCH2, pp)));
      }
    } else {
#pragma unroll
      for (int i = 0; i < H; i++) nz2[i] = f2_pack(-y[2 * i], -y[2 * i + 1]);
    }
#pragma unroll
    for (int i = 0; i < H; i++) {
      float a, b;
      f2_unpack(nz2[i], a, b);
      xf[2 * i] = fminf(fmaxf(a, -18.0f), 88.75f);   // a NaN becomes -18: the final product restores it
      xf[2 * i + 1] = fminf(fmaxf(b, -18.0f), 88.75f);
    }
  }
#pragma unroll
  for (int i = 0; i < H; i++) {
    const uint64_t x2 = f2_pack(xf[2 * i], xf[2 * i + 1]);
    const uint64_t t2 = f2_fma(x2, f2_dup(256.0f), MAG2);
    c2[i] = f2_fma(f2_sub(t2, MAG2), f2_dup(-0.00390625f), x2);
    float ta, tb;
    f2_unpack(t2, ta, tb);
    k[2 * i] = __float_as_int(ta) - 0x4B400000;
    k[2 * i + 1] = __float_as_int(tb) - 0x4B400000;
  }
  {
    uint64_t p2[H], tl2[H], qr2[H];
    const float* t1 = tbl - EXP_FF_A_MIN;
    const float* t2 = tbl + EXP_FF_A_COUNT;
#pragma unroll
    for (int i = 0; i < H; i++) {
      const int a0 = k[2 * i] >> 8, a1 = k[2 * i + 1] >> 8, b0 = k[2 * i] & 255, b1 = k[2 * i + 1] & 255;
      const uint64_t h1 = f2_pack(t1[a0], t1[a1]), l1 = f2_pack(t1[EXP_FF_ENTRIES + a0], t1[EXP_FF_ENTRIES + a1]);
      const uint64_t hh = f2_pack(t2[b0], t2[b1]), ll = f2_pack(t2[EXP_FF_ENTRIES + b0], t2[EXP_FF_ENTRIES + b1]);
      p2[i] = f2_mul(h1, hh);
      const uint64_t pn = f2_mul(p2[i], f2_dup(-1.0f));
      tl2[i] = f2_fma(h1, ll, f2_fma(l1, hh, f2_fma(h1, hh, pn)));
    }
#pragma unroll
    for (int i = 0; i < H; i++) {
      const uint64_t w = f2_fma(c2[i], f2_fma(c2[i], f2_dup(1.0f / 24.0f), f2_dup(1.0f / 6.0f)), f2_dup(0.5f));
      qr2[i] = f2_mul(f2_mul(c2[i], c2[i]), w);
    }
#pragma unroll
    for (int i = 0; i < H; i++) {
      const uint64_t u = f2_mul(p2[i], c2[i]);
      const uint64_t un = f2_mul(u, f2_dup(-1.0f));
      const uint64_t lo = f2_add(f2_fma(p2[i], qr2[i], f2_fma(p2[i], c2[i], un)), f2_fma(tl2[i], c2[i], tl2[i]));
      h2[i] = f2_add(p2[i], u);
      low2[i] = f2_add(f2_sub(u, f2_sub(h2[i], p2[i])), lo);
    }
  }
  bool uncertain = false;
#pragma unroll
  for (int i = 0; i < H; i++) {
    const uint64_t e2 = f2_add(h2[i], f2_fma(h2[i], f2_dup(3.637978807091713e-12f), low2[i]));   // low +- 2^-38 h
    const uint64_t f2 = f2_add(h2[i], f2_fma(h2[i], f2_dup(-3.637978807091713e-12f), low2[i]));
    f2_unpack(e2, ea[2 * i], ea[2 * i + 1]);
    f2_unpack(f2, eb[2 * i], eb[2 * i + 1]);
    // Arguments from the overflow threshold on (exp rounds to +Inf, the sigmoid is 0) may have produced Inf - Inf above:
    // they are settled by the comparison with the threshold alone.
    uncertain |= ((ea[2 * i] != eb[2 * i]) & (xf[2 * i] < EXP_OVERFLOW_F)) | ((ea[2 * i + 1] != eb[2 * i + 1]) & (xf[2 * i + 1] < EXP_OVERFLOW_F));
    nd2[i] = f2_sub(f2_dup(-1.0f), e2);                                  // -(1 + e), the same rounding
    nds2[i] = f2_mul(nd2[i], f2_dup(2.3283064365386963e-10f));
  }
#pragma unroll
  for (int i = 0; i < H; i++) {
    float a, b;
    f2_unpack(nds2[i], a, b);
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(g[2 * i]) : "f"(-a));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(g[2 * i + 1]) : "f"(-b));
  }
#pragma unroll
  for (int i = 0; i < H; i++) {
    uint64_t gg = f2_pack(g[2 * i], g[2 * i + 1]);
    gg = f2_fma(gg, f2_fma(nds2[i], gg, ONE2), gg);
    g2[i] = f2_mul(gg, f2_dup(2.3283064365386963e-10f));
    f2_unpack(g2[i], g[2 * i], g[2 * i + 1]);
    f2_unpack(f2_fma(nd2[i], g2[i], ONE2), res[2 * i], res[2 * i + 1]);
  }
#pragma unroll
  for (int i = 0; i < W; i++) cand[i] = __int_as_float(__float_as_int(g[i]) + (res[i] > 0.0f ? 1 : -1));
#pragma unroll
  for (int i = 0; i < H; i++) f2_unpack(f2_fma(nd2[i], f2_pack(cand[2 * i], cand[2 * i + 1]), ONE2), rc[2 * i], rc[2 * i + 1]);
#pragma unroll
  for (int i = 0; i < W; i++) {
    const float best = (fabsf(rc[i]) < fabsf(res[i])) ? cand[i] : g[i];
    sg[i] = (xf[i] < EXP_OVERFLOW_F) ? best : 0.0f;
  }
  if (__any_sync(0xffffffffu, uncertain)) {   // about one warp-call in forty: those lanes redo their eight in binary64
    if (uncertain) {
      const double* dtbl = reinterpret_cast<const double*>(kExp2TableBits);   // global memory: rare enough
#pragma unroll
      for (int i = 0; i < W; i++) sg[i] = sigmoid_fast((ACT_T == ACT_GELU_SIGMOID) ? mul_1702(y[i]) : y[i], dtbl);
    }
  }
#pragma unroll
  for (int i = 0; i < H; i++) f2_unpack(f2_mul(f2_pack(y[2 * i], y[2 * i + 1]), f2_pack(sg[2 * i], sg[2 * i + 1])), y[2 * i], y[2 * i + 1]);
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
