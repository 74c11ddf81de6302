// CPU oracle for the int8 quantized-inference path of slexisvn/mlfw (v0.1.6).
//
// THIS FILE IS TEST INFRASTRUCTURE.  It is a plain C++ restatement of the
// arithmetic the reference's TypeScript CPU target performs, written so that
// the CUDA backend can be checked against it.  Only the tests, the smoke check
// and the CPU-baseline leg of the benchmark may call it; the product never does.
//
// Parity pin: the reference is TypeScript and no JavaScript engine exists in
// the build image, so the reference itself cannot be run.  The oracle is pinned
// against every closed-form known answer the reference's own tests hold for
// this path (tests/compiler/passes/quantization/params.test.js, pass.test.js,
// tests/e2e/cuda/training-quant.cuda.test.js): those are restated in
// tests/test_oracle_reference_vectors.py.  Behaviour the reference's tests do
// not pin (exact ties, NaN/Inf input, tanh-GELU) follows the reference SOURCE
// and is marked "source-only" where it is restated below.
//
// Reference files restated (paths inside the reference project):
//   src/compiler/ir/graph/quantization_types.ts   QuantizationParams  ("mode P", all binary64)
//   src/compiler/passes/lowering/quant_math.ts     quantize/dequantize leaf math ("mode C")
//   src/compiler/passes/lowering/rules/quantization.ts   quantized_dot
//   src/backend/cpu/codegen.ts                      where Math.fround / Math.round / |0 land
//   src/compiler/passes/quantization/quantization_pass.ts:390-459  per-channel tail
//   src/compiler/passes/decompose/decomposition_pass.ts:197-230    sigmoid, gelu(1.702), silu
//   src/compiler/analysis/calibration.ts           min/max observer
//   src/compiler/passes/decompose/decomposition_pass.ts:156-174, 232-260 and src/nn/functional/attention.ts:42-74
//                                                   softmax, layer_norm, attention (tolerance only)
//   src/util/random.ts, src/tensor/factory/creation_ops.ts, src/nn/init.ts  seeded data
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// ---------------------------------------------------------------------------
// ECMAScript number semantics
// ---------------------------------------------------------------------------

// Math.round: nearest integer, ties toward +infinity; NaN and +-Inf pass through.
// floor(x) and x - floor(x) are exact in binary64, so this is the spec's rule.
inline double js_round(double x) {
  if (!std::isfinite(x)) return x;
  double r = std::floor(x);
  if (x - r >= 0.5) r += 1.0;
  return r;
}

// Math.fround: binary64 -> binary32 (round to nearest even) -> binary64.
inline double js_fround(double v) { return (double)(float)v; }

// Math.max / Math.min: NaN if either argument is NaN.
inline double js_max(double a, double b) {
  if (std::isnan(a) || std::isnan(b)) return std::numeric_limits<double>::quiet_NaN();
  return a > b ? a : b;
}
inline double js_min(double a, double b) {
  if (std::isnan(a) || std::isnan(b)) return std::numeric_limits<double>::quiet_NaN();
  return a < b ? a : b;
}

// ToInt32: NaN/Inf -> 0, otherwise truncate and wrap modulo 2^32.
inline int32_t js_to_int32(double v) {
  if (!std::isfinite(v)) return 0;
  double t = std::trunc(v);
  double m = std::fmod(t, 4294967296.0);
  if (m < 0) m += 4294967296.0;
  return (int32_t)(uint32_t)m;
}
// Store into Int8Array / Uint8Array: ToInt32 then keep the low 8 bits.
inline int8_t js_to_int8(double v) { return (int8_t)(uint8_t)(uint32_t)js_to_int32(v); }

// x || fallback  (0, -0 and NaN are falsy)
inline double js_or(double x, double fallback) { return (x == 0.0 || std::isnan(x)) ? fallback : x; }

// ---------------------------------------------------------------------------
// Seeded data: src/util/random.ts:5-14 (mulberry32)
// ---------------------------------------------------------------------------
struct Mulberry32 {
  uint32_t a;
  explicit Mulberry32(uint32_t seed) : a(seed) {}
  double next() {
    a += 0x6d2b79f5u;
    uint32_t t = (a ^ (a >> 15)) * (1u | a);
    t = (t + ((t ^ (t >> 7)) * (61u | t))) ^ t;
    return (double)(t ^ (t >> 14)) / 4294967296.0;
  }
};

enum { SCHEME_SYM = 0, SCHEME_ASYM = 1, SCHEME_PER_CHANNEL = 2 };
enum { DT_I8 = 0, DT_UI8 = 1 };

// quantization_types.ts:62-73
inline void clamp_range(int scheme, int dtype, int numBits, double* cMin, double* cMax) {
  if (scheme == SCHEME_SYM) {
    double b = std::ldexp(1.0, numBits - 1) - 1.0;
    *cMin = -b; *cMax = b; return;
  }
  if (dtype == DT_UI8) { *cMin = 0; *cMax = std::ldexp(1.0, numBits) - 1.0; return; }
  *cMin = -std::ldexp(1.0, numBits - 1);
  *cMax = std::ldexp(1.0, numBits - 1) - 1.0;
}

// quantization_types.ts:75-79 (also the body of quantizeArray / quantizeArrayPerChannel)
inline double qp_quantize(double x, double scale, double zp, double cMin, double cMax) {
  double raw = js_round(x / scale + zp);
  return js_max(cMin, js_min(cMax, raw));
}

enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU_SIGMOID = 2, ACT_GELU_TANH = 3, ACT_SILU = 4 };

// decomposition_pass.ts:197-203 evaluated by the CPU target: every f32 binary
// op is computed in binary64 and rounded once (cpu/codegen.ts:496); exp is
// Math.exp in binary64, then rounded (cpu/codegen.ts:532-534).
inline float sigmoid_ref(float z) {
  float e = (float)std::exp((double)(-z));
  float d = (float)(1.0 + (double)e);
  return (float)(1.0 / (double)d);
}

inline float activation_ref(float y, int act) {
  switch (act) {
    case ACT_NONE: return y;
    case ACT_RELU: {  // builder.ts:561-565: maximum(x, 0) -> Math.max
      double m = js_max((double)y, 0.0);
      return (float)m;
    }
    case ACT_GELU_SIGMOID: {  // decomposition_pass.ts:212-222: x * sigmoid(1.702 x); 1.702 is a binary64 immediate
      float z = (float)(1.702 * (double)y);
      return (float)((double)y * (double)sigmoid_ref(z));
    }
    case ACT_SILU:  // decomposition_pass.ts:224-230
      return (float)((double)y * (double)sigmoid_ref(y));
    case ACT_GELU_TANH: {
      // No reference implementation exists (the reference's gelu is the sigmoid
      // form above).  Standard tanh form, each binary op rounded to binary32,
      // tanh computed in binary64 then rounded, constants as binary64 immediates.
      float y2 = (float)((double)y * (double)y);
      float y3 = (float)((double)y2 * (double)y);
      float c = (float)(0.044715 * (double)y3);
      float in = (float)((double)y + (double)c);
      float u = (float)(0.7978845608028654 * (double)in);
      float t = (float)std::tanh((double)u);
      float o = (float)(1.0 + (double)t);
      float h = (float)(0.5 * (double)y);
      return (float)((double)h * (double)o);
    }
  }
  return y;
}

}  // namespace

extern "C" {

// --------------------------- seeded data -----------------------------------

void orc_rng_uniform(uint32_t seed, int64_t n, double* out) {
  Mulberry32 g(seed);
  for (int64_t i = 0; i < n; i++) out[i] = g.next();
}

// nn/init.ts:40-53 normal_ (== creation_ops.ts:61-75 randn when mean 0, std 1); stored to Float32Array.
void orc_normal_f32(uint32_t seed, int64_t n, double mean, double stdv, float* out) {
  Mulberry32 g(seed);
  for (int64_t i = 0; i < n; i += 2) {
    double u1 = js_or(g.next(), 1e-10);
    double u2 = g.next();
    double r = std::sqrt(-2.0 * std::log(u1));
    double theta = 6.283185307179586 * u2;
    out[i] = (float)(mean + stdv * r * std::cos(theta));
    if (i + 1 < n) out[i + 1] = (float)(mean + stdv * r * std::sin(theta));
  }
}

// nn/init.ts:31-38 uniform_
void orc_uniform_f32(uint32_t seed, int64_t n, double a, double b, float* out) {
  Mulberry32 g(seed);
  double range = b - a;
  for (int64_t i = 0; i < n; i++) out[i] = (float)(a + g.next() * range);
}

// Integer weights uniform in [lo, hi]: floor(u * (hi-lo+1)) + lo (util/random.ts:36-38 randomInt).
void orc_randint_i8(uint32_t seed, int64_t n, int lo, int hi, int8_t* out) {
  Mulberry32 g(seed);
  double span = (double)(hi - lo + 1);
  for (int64_t i = 0; i < n; i++) out[i] = (int8_t)((int)std::floor(g.next() * span) + lo);
}

// --------------------------- QuantizationParams ----------------------------

void orc_qp_clamp_range(int scheme, int dtype, int numBits, double* cMin, double* cMax) {
  clamp_range(scheme, dtype, numBits, cMin, cMax);
}

// quantization_types.ts:241-264 fromRange
void orc_qp_from_range(double mn, double mx, int scheme, int dtype, int numBits, double* scale, double* zp) {
  if (scheme == SCHEME_SYM) {
    double absMax = std::fmax(std::fabs(mn), std::fabs(mx));
    double bound = std::ldexp(1.0, numBits - 1) - 1.0;
    *scale = js_or(absMax / bound, 1e-10);
    *zp = 0;
    return;
  }
  double cMin, cMax;
  if (dtype == DT_UI8) { cMin = 0; cMax = std::ldexp(1.0, numBits) - 1.0; }
  else { cMin = -std::ldexp(1.0, numBits - 1); cMax = std::ldexp(1.0, numBits - 1) - 1.0; }
  double range = js_or(mx - mn, 1e-10);
  *scale = range / (cMax - cMin);
  double z = js_round(cMin - mn / *scale);
  *zp = js_max(cMin, js_min(cMax, z));
}

// quantization_types.ts:287-297 fromConstantArray
void orc_qp_from_constant_array(const double* data, int64_t n, int scheme, int dtype, int numBits,
                                double* scale, double* zp) {
  double mn = INFINITY, mx = -INFINITY;
  for (int64_t i = 0; i < n; i++) {
    if (data[i] < mn) mn = data[i];
    if (data[i] > mx) mx = data[i];
  }
  if (!std::isfinite(mn)) mn = -1;
  if (!std::isfinite(mx)) mx = 1;
  if (mn == mx) { mn -= 0.5; mx += 0.5; }
  orc_qp_from_range(mn, mx, scheme, dtype, numBits, scale, zp);
}

double orc_qp_quantize(double x, double scale, double zp, double cMin, double cMax) {
  return qp_quantize(x, scale, zp, cMin, cMax);
}
double orc_qp_dequantize(double q, double scale, double zp) { return (q - zp) * scale; }

// quantization_types.ts:299-317 + 266-281: per-channel symmetric scales for a
// tensor viewed as [outer, numCh, stride] (stride = product of dims after axis).
#define ORC_PER_CHANNEL_SCALES(NAME, T)                                                          \
  void NAME(const T* data, int64_t outer, int64_t numCh, int64_t stride, int numBits,            \
            double* scales) {                                                                    \
    std::vector<double> mins(numCh, INFINITY), maxs(numCh, -INFINITY);                           \
    for (int64_t o = 0; o < outer; o++)                                                          \
      for (int64_t c = 0; c < numCh; c++) {                                                      \
        const T* p = data + (o * numCh + c) * stride;                                            \
        double mn = mins[c], mx = maxs[c];                                                       \
        for (int64_t s = 0; s < stride; s++) {                                                   \
          double v = (double)p[s];                                                               \
          if (v < mn) mn = v;                                                                    \
          if (v > mx) mx = v;                                                                    \
        }                                                                                        \
        mins[c] = mn; maxs[c] = mx;                                                              \
      }                                                                                          \
    double bound = std::ldexp(1.0, numBits - 1) - 1.0;                                           \
    for (int64_t c = 0; c < numCh; c++) {                                                        \
      double mn = mins[c], mx = maxs[c];                                                         \
      if (!std::isfinite(mn)) mn = -1;                                                           \
      if (!std::isfinite(mx)) mx = 1;                                                            \
      if (mn == mx) { mn -= 0.5; mx += 0.5; }                                                    \
      double absMax = std::fmax(std::fabs(mn), std::fabs(mx));                                   \
      scales[c] = js_or(absMax / bound, 1e-10);                                                  \
    }                                                                                            \
  }
ORC_PER_CHANNEL_SCALES(orc_per_channel_scales_f32, float)
ORC_PER_CHANNEL_SCALES(orc_per_channel_scales_f64, double)

// quantization_types.ts:118-130 quantizeArrayPerChannel.  Codes are returned as
// doubles (they may be NaN) and, separately, as they land in an Int8Array.
#define ORC_QUANT_PER_CHANNEL(NAME, T)                                                           \
  void NAME(const T* data, int64_t outer, int64_t numCh, int64_t stride, const double* scales,   \
            double cMin, double cMax, int8_t* q8, double* qd) {                                  \
    _Pragma("omp parallel for collapse(2) schedule(static)")                                     \
    for (int64_t o = 0; o < outer; o++)                                                          \
      for (int64_t c = 0; c < numCh; c++) {                                                      \
        int64_t base = (o * numCh + c) * stride;                                                 \
        double sc = scales[c];                                                                   \
        for (int64_t s = 0; s < stride; s++) {                                                   \
          double q = qp_quantize((double)data[base + s], sc, 0.0, cMin, cMax);                   \
          if (q8) q8[base + s] = js_to_int8(q);                                                  \
          if (qd) qd[base + s] = q;                                                              \
        }                                                                                        \
      }                                                                                          \
  }
ORC_QUANT_PER_CHANNEL(orc_quantize_per_channel_f32, float)
ORC_QUANT_PER_CHANNEL(orc_quantize_per_channel_f64, double)

// quantization_types.ts:132-141 dequantizeArrayPerChannel (binary64 result).
void orc_dequantize_per_channel(const int8_t* q, int64_t outer, int64_t numCh, int64_t stride,
                                const double* scales, double* out) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t o = 0; o < outer; o++)
    for (int64_t c = 0; c < numCh; c++) {
      int64_t base = (o * numCh + c) * stride;
      for (int64_t s = 0; s < stride; s++) out[base + s] = ((double)q[base + s] - 0.0) * scales[c];
    }
}

// Per-token activation quantization = fromConstantArrayPerChannel(x, [M,K], axis 0)
// + quantizeArrayPerChannel; scales64 keeps the reference's binary64 scales,
// scales32 is what the device interface carries (Float32Array store of the same number).
void orc_quantize_per_token(const float* x, int64_t M, int64_t K, double cMin, double cMax,
                            int8_t* q, double* scales64, float* scales32) {
  std::vector<double> sc(M);
  orc_per_channel_scales_f32(x, 1, M, K, 8, sc.data());
  orc_quantize_per_channel_f32(x, 1, M, K, sc.data(), cMin, cMax, q, nullptr);
  for (int64_t m = 0; m < M; m++) {
    if (scales64) scales64[m] = sc[m];
    if (scales32) scales32[m] = (float)sc[m];
  }
}

// Device-interface dequantize: y = fround(q * (double)scale32[m]).
void orc_dequantize_per_token_f32(const int8_t* q, const float* scales32, int64_t M, int64_t K, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++)
    for (int64_t k = 0; k < K; k++) y[m * K + k] = (float)((double)q[m * K + k] * (double)scales32[m]);
}

// --------------------------- compiled ops (mode C) -------------------------

// quant_math.ts:16-27 as emitted by cpu/codegen.ts: fround(x / scale) [fround(+zp)]
// -> Math.round -> Math.max(cMin) -> Math.min(cMax) -> (v|0) -> Int8Array/Uint8Array store.
void orc_quantize_static(const float* x, int64_t n, double scale, double zp, int dtype, int8_t* out) {
  double cMin = dtype == DT_UI8 ? 0 : -128, cMax = dtype == DT_UI8 ? 255 : 127;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    double t = js_fround((double)x[i] / scale);
    if (zp != 0) t = js_fround(t + zp);
    double r = js_round(t);
    double c = js_min(js_max(r, cMin), cMax);
    out[i] = js_to_int8((double)js_to_int32(c));
  }
}

// quant_math.ts:29-34: (+q) [fround(- zp)] then fround(* scale).  The int->f32
// cast is emitted as (+x), i.e. NOT rounded to binary32 (cpu/codegen.ts:521).
void orc_dequantize_static_i8(const int8_t* q, int64_t n, double scale, double zp, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    double v = (double)q[i];
    if (zp != 0) v = js_fround(v - zp);
    y[i] = (float)(v * scale);
  }
}
void orc_dequantize_static_u8(const uint8_t* q, int64_t n, double scale, double zp, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    double v = (double)q[i];
    if (zp != 0) v = js_fround(v - zp);
    y[i] = (float)(v * scale);
  }
}
void orc_dequantize_static_i32(const int32_t* q, int64_t n, double scale, double zp, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) {
    double v = (double)q[i];
    if (zp != 0) v = js_fround(v - zp);
    y[i] = (float)(v * scale);
  }
}

// rules/quantization.ts:23-42: C[m,n] = sum_k (A[m,k]-zpA) * (B-zpB), accumulated
// exactly (binary64 in JS; all partial sums are integers below 2^53) and stored
// to an Int32Array (ToInt32 wrap).  w_layout 0: W is [N,K] (contract dim 1);
// 1: W is [K,N] (contract dim 0).  threads <= 0 means all cores.
void orc_qdot_i32(const int8_t* A, const int8_t* W, int64_t M, int64_t N, int64_t K, int w_layout,
                  int zpA, int zpB, int32_t* C, int threads) {
#ifdef _OPENMP
  int nt = threads > 0 ? threads : omp_get_max_threads();
#else
  int nt = 1;
#endif
  (void)nt;
  std::vector<int8_t> wt;
  const int8_t* Wnk = W;
  if (w_layout == 1) {  // make K contiguous once; the arithmetic does not change
    wt.resize((size_t)N * K);
    for (int64_t k = 0; k < K; k++)
      for (int64_t n = 0; n < N; n++) wt[(size_t)n * K + k] = W[(size_t)k * N + n];
    Wnk = wt.data();
  }
#pragma omp parallel for schedule(static) num_threads(nt)
  for (int64_t m = 0; m < M; m++) {
    const int8_t* a = A + m * K;
    for (int64_t n = 0; n < N; n++) {
      const int8_t* w = Wnk + n * K;
      int64_t acc = 0;
      if (zpA == 0 && zpB == 0) {
        int32_t acc32 = 0;  // exact while K*128*128 < 2^31 (K < 131072); chunked to be safe
        for (int64_t k0 = 0; k0 < K; k0 += 65536) {
          int64_t k1 = k0 + 65536 < K ? k0 + 65536 : K;
          acc32 = 0;
          for (int64_t k = k0; k < k1; k++) acc32 += (int32_t)a[k] * (int32_t)w[k];
          acc += acc32;
        }
      } else {
        for (int64_t k = 0; k < K; k++) acc += (int64_t)((int)a[k] - zpA) * (int64_t)((int)w[k] - zpB);
      }
      C[m * N + n] = (int32_t)(uint32_t)(uint64_t)acc;  // ToInt32 wrap
    }
  }
}

// Per-channel tail (quantization_pass.ts:427-456) + bias (nn/functional/linear.ts:13-15)
// + activation, in the fused-region form the CPU target evaluates:
//   sv   = fround(aScale * wScale[n])          (binary64 product stored as an f32 constant)
//   t    = fround((+acc) * sv)                 (int->f32 cast is not rounded)
//   y    = fround(t + bias[n])
//   out  = act(y)
// a_scales has M entries when per_token != 0 (the per-token extension: the same
// expression with aScale varying per row), else one entry.
void orc_epilogue(const int32_t* acc, int64_t M, int64_t N, const float* a_scales, int per_token,
                  const float* w_scales, const float* bias, int act, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    double as = (double)a_scales[per_token ? m : 0];
    for (int64_t n = 0; n < N; n++) {
      float sv = (float)(as * (double)w_scales[n]);
      float t = (float)((double)acc[m * N + n] * (double)sv);
      float y = bias ? (float)((double)t + (double)bias[n]) : t;
      out[m * N + n] = activation_ref(y, act);
    }
  }
}

// Same tail when the scale vector is given directly (static activation scale:
// sv[n] = fround(aScale64 * wScale64[n]) is formed by the caller in binary64).
void orc_epilogue_sv(const int32_t* acc, int64_t M, int64_t N, const float* sv, const float* bias, int act,
                     float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++)
    for (int64_t n = 0; n < N; n++) {
      float t = (float)((double)acc[m * N + n] * (double)sv[n]);
      float y = bias ? (float)((double)t + (double)bias[n]) : t;
      out[m * N + n] = activation_ref(y, act);
    }
}

void orc_activation(const float* y, int64_t n, int act, float* out) {
  for (int64_t i = 0; i < n; i++) out[i] = activation_ref(y[i], act);
}

// calibration.ts:11-39 min/max observer (NaN never wins a strict comparison).
void orc_minmax_observe(const float* x, int64_t n, double* mn, double* mx) {
  double a = *mn, b = *mx;
  for (int64_t i = 0; i < n; i++) {
    double v = (double)x[i];
    if (v < a) a = v;
    if (v > b) b = v;
  }
  *mn = a; *mx = b;
}

// ---------------------------------------------------------------------------
// f32 pieces of a transformer block (the "next" components around the int8 linears).
// Each operation of the decomposed graph is a binary32 operation (binary64 then
// Math.fround); reductions add the elements in index order.  The reference can lower
// these through more than one path (fused or not, different loop nests), and its
// tests only bound them by tolerances, so the device results are compared with this
// restatement to a tolerance as well -- never bit for bit.
// ---------------------------------------------------------------------------

// layer_norm: src/compiler/passes/decompose/decomposition_pass.ts:232-260
//   mean = reduce_mean(x); c = x - mean; var = reduce_mean(c * c); r = rsqrt(var + eps);
//   y = c * r * gamma + beta.  `add` (optional) is summed to x first (ops.add of the residual stream).
void orc_layer_norm(const float* x, const float* add, const float* gamma, const float* beta, double eps, int64_t M, int64_t D,
                    float* sum_out, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; m++) {
    std::vector<float> row((size_t)D);
    for (int64_t d = 0; d < D; d++) {
      float v = x[m * D + d];
      if (add) v = (float)((double)v + (double)add[m * D + d]);
      row[(size_t)d] = v;
      if (sum_out) sum_out[m * D + d] = v;
    }
    float acc = 0.0f;
    for (int64_t d = 0; d < D; d++) acc = (float)((double)acc + (double)row[(size_t)d]);
    const float mean = (float)((double)acc / (double)D);
    float acc2 = 0.0f;
    for (int64_t d = 0; d < D; d++) {
      const float c = (float)((double)row[(size_t)d] - (double)mean);
      row[(size_t)d] = c;
      acc2 = (float)((double)acc2 + (double)(float)((double)c * (double)c));
    }
    const float var = (float)((double)acc2 / (double)D);
    const float ve = (float)((double)var + (double)(float)eps);
    const float r = (float)(1.0 / std::sqrt((double)ve));
    for (int64_t d = 0; d < D; d++) {
      const float n = (float)((double)row[(size_t)d] * (double)r);
      const float g = (float)((double)n * (double)gamma[d]);
      y[m * D + d] = (float)((double)g + (double)beta[d]);
    }
  }
}

// scaled_dot_product_attention: src/nn/functional/attention.ts:42-74 with the softmax of
// src/compiler/passes/decompose/decomposition_pass.ts:156-174.
//   scores = matmul(q, k^T) * scale (+ mask: 0 where j <= i + S - L, else -Infinity);
//   w = exp(scores - max) / sum(exp(scores - max)); out = matmul(w, v).
// Row (b, s) of head h starts at base + (b*S + s)*ld + h*Dh.  `rows` (optional) lists the flattened
// (b*H + h)*S + i query rows to compute, so that large cases can be spot checked.
void orc_sdpa(const float* q, const float* k, const float* v, int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t B, int64_t H,
              int64_t S, int64_t Dh, double scale, int causal, const int64_t* rows, int64_t nrows, float* out, int64_t ld_o) {
  const int64_t total = rows ? nrows : B * H * S;
  const float scale32 = (float)scale;
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t t = 0; t < total; t++) {
    const int64_t flat = rows ? rows[t] : t;
    const int64_t i = flat % S, bh = flat / S, h = bh % H, b = bh / H;
    const float* qi = q + (b * S + i) * ld_q + h * Dh;
    std::vector<float> sc((size_t)S);
    float mx = -std::numeric_limits<float>::infinity();
    for (int64_t j = 0; j < S; j++) {
      const float* kj = k + (b * S + j) * ld_k + h * Dh;
      float acc = 0.0f;
      for (int64_t d = 0; d < Dh; d++) acc = (float)((double)acc + (double)(float)((double)qi[d] * (double)kj[d]));
      float sv = (float)((double)acc * (double)scale32);
      if (causal) sv = (float)((double)sv + (j <= i ? 0.0 : -std::numeric_limits<double>::infinity()));
      sc[(size_t)j] = sv;
      if (sv > mx) mx = sv;
    }
    float sum = 0.0f;
    for (int64_t j = 0; j < S; j++) {
      const float e = (float)std::exp((double)(float)((double)sc[(size_t)j] - (double)mx));
      sc[(size_t)j] = e;
      sum = (float)((double)sum + (double)e);
    }
    // rows == null writes in place of the inputs' layout; a row list writes densely: row t of [nrows, Dh]
    float* o = rows ? out + t * ld_o : out + (b * S + i) * ld_o + h * Dh;
    for (int64_t d = 0; d < Dh; d++) {
      float acc = 0.0f;
      for (int64_t j = 0; j < S; j++) {
        const float w = (float)((double)sc[(size_t)j] / (double)sum);
        acc = (float)((double)acc + (double)(float)((double)w * (double)v[(b * S + j) * ld_v + h * Dh + d]));
      }
      o[d] = acc;
    }
  }
}

// ---------------------------------------------------------------------------
// Per-group quantization (GPTQ / AWQ-style INT4): quantization_types.ts:319-340
// (fromConstantArrayPerGroup), :143-153 (quantizeArrayPerGroup), :155-162
// (dequantizeArrayPerGroup).  Groups are runs of groupSize consecutive elements of
// the flat array (the last one may be shorter); zero-points are 0; the scheme is
// not the symmetric one, so the clamp is [-2^(b-1), 2^(b-1)-1] (:62-73).
// ---------------------------------------------------------------------------
#define ORC_PER_GROUP_SCALES(NAME, T)                                                            \
  void NAME(const T* data, int64_t n, int64_t groupSize, int numBits, double* scales) {          \
    const int64_t groups = (n + groupSize - 1) / groupSize;                                      \
    const double bound = std::ldexp(1.0, numBits - 1) - 1.0;                                     \
    _Pragma("omp parallel for schedule(static)")                                                 \
    for (int64_t g = 0; g < groups; g++) {                                                       \
      const int64_t start = g * groupSize, end = std::min(start + groupSize, n);                 \
      double absMax = 0;                                                                         \
      for (int64_t i = start; i < end; i++) {                                                    \
        double a = std::fabs((double)data[i]);                                                   \
        if (a > absMax) absMax = a;                                                              \
      }                                                                                          \
      scales[g] = js_or(absMax / bound, 1e-10);                                                  \
    }                                                                                            \
  }
ORC_PER_GROUP_SCALES(orc_per_group_scales_f32, float)
ORC_PER_GROUP_SCALES(orc_per_group_scales_f64, double)

#define ORC_QUANT_PER_GROUP(NAME, T)                                                             \
  void NAME(const T* data, int64_t n, int64_t groupSize, int numBits, const double* scales,      \
            int8_t* q8, double* qd) {                                                            \
    const double cMin = -std::ldexp(1.0, numBits - 1), cMax = std::ldexp(1.0, numBits - 1) - 1.0; \
    _Pragma("omp parallel for schedule(static)")                                                 \
    for (int64_t i = 0; i < n; i++) {                                                            \
      double q = qp_quantize((double)data[i], scales[i / groupSize], 0.0, cMin, cMax);           \
      if (q8) q8[i] = js_to_int8(q);                                                             \
      if (qd) qd[i] = q;                                                                         \
    }                                                                                            \
  }
ORC_QUANT_PER_GROUP(orc_quantize_per_group_f32, float)
ORC_QUANT_PER_GROUP(orc_quantize_per_group_f64, double)

void orc_dequantize_per_group(const int8_t* q, int64_t n, int64_t groupSize, const double* scales, double* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; i++) out[i] = ((double)q[i] - 0.0) * scales[i / groupSize];
}

// ---------------------------------------------------------------------------
// quantized_conv, two spatial dimensions: ops/quantization.ts:156-190, lowering
// rules/quantization.ts:44-62 over the loop nest of lowering_registry.ts:335-449.
//   out[n,oc,oh,ow] = sum_{ic,kh,kw} inside ? (in[n, g*Cg+ic, ih, iw] - zpIn) * (ker[oc,ic,kh,kw] - zpKer) : 0
//   ih = oh*sh + kh*dh - padTop, iw = ow*sw + kw*dw - padLeft, g = oc / (O / groups)
// A tap outside the input adds 0 (the guard's fill), not (0 - zpIn) * (...).  The accumulator is an Int32Array
// element: every addition is stored back with ToInt32.  Output extents follow ops/linalg.ts:236-246.
// layout 0: input / output NCHW, kernel OIHW;  1: input / output NHWC, kernel OHWI.
// ---------------------------------------------------------------------------
void orc_quantized_conv2d(const int8_t* in, const int8_t* ker, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                          int64_t KH, int64_t KW, int sh, int sw, int padTop, int padBottom, int padLeft, int padRight,
                          int dh, int dw, int groups, int zpIn, int zpKer, int layout, int32_t* out) {
  const int64_t OH = (H + padTop + padBottom - ((KH - 1) * dh + 1)) / sh + 1;
  const int64_t OW = (W + padLeft + padRight - ((KW - 1) * dw + 1)) / sw + 1;
  const int64_t Cg = C / groups, Og = O / groups;
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t n = 0; n < N; n++)
    for (int64_t oc = 0; oc < O; oc++) {
      const int64_t g = oc / Og;
      for (int64_t oh = 0; oh < OH; oh++)
        for (int64_t ow = 0; ow < OW; ow++) {
          int32_t acc = 0;
          for (int64_t ic = 0; ic < Cg; ic++)
            for (int64_t kh = 0; kh < KH; kh++)
              for (int64_t kw = 0; kw < KW; kw++) {
                const int64_t ih = oh * sh + kh * dh - padTop, iw = ow * sw + kw * dw - padLeft;
                if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                const int64_t c = g * Cg + ic;
                const int64_t ii = layout == 0 ? ((n * C + c) * H + ih) * W + iw : ((n * H + ih) * W + iw) * C + c;
                const int64_t ki = layout == 0 ? ((oc * Cg + ic) * KH + kh) * KW + kw : ((oc * KH + kh) * KW + kw) * Cg + ic;
                const double prod = (double)((int)in[ii] - zpIn) * (double)((int)ker[ki] - zpKer);
                acc = js_to_int32((double)acc + prod);
              }
          const int64_t oi = layout == 0 ? ((n * O + oc) * OH + oh) * OW + ow : ((n * OH + oh) * OW + ow) * O + oc;
          out[oi] = acc;
        }
    }
}

double orc_js_round(double x) { return js_round(x); }
// The benchmark's CPU arm runs under launchers that export OMP_NUM_THREADS=1; it asks for the cores it may use.
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}
int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"
