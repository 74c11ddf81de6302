// koffi binding of libb200q.so — the C ABI declared in include/b200q.h.
// Same idiom as the reference's terac binding (src/runtime/node/terac.ts:88-101):
// koffi.load + lib.func('<C prototype>'), one cached binding per library path.
// This file is source only in this repository: no JavaScript engine exists in the
// build image, so it is exercised through its Python twin (mlfw_b200/_lib.py).
import koffi from 'koffi';

export type B200QBinding = ReturnType<typeof bind>;

let cached: { path: string; binding: B200QBinding } | null = null;

function bind(path: string) {
  const lib = koffi.load(path);
  const f = (proto: string) => lib.func(proto);
  return {
    deviceCount: f('int b200q_device_count()'),
    create: f('int b200q_create(int device, _Out_ void **ctx)'),
    destroy: f('void b200q_destroy(void *ctx)'),
    lastError: f('str b200q_last_error()'),
    sync: f('int b200q_sync(void *ctx)'),
    statusWord: f('int b200q_status_word(void *ctx, _Out_ uint32_t *word)'),
    alloc: f('int b200q_alloc(void *ctx, size_t bytes, _Out_ void **dev)'),
    free: f('int b200q_free(void *ctx, void *dev)'),
    upload: f('int b200q_upload(void *ctx, void *dev, const void *host, size_t bytes)'),
    download: f('int b200q_download(void *ctx, void *host, const void *dev, size_t bytes)'),
    quantizePerToken: f('int b200q_quantize_per_token(void *ctx, const void *x, int64_t M, int64_t K, void *q, void *scales, int qmin, int qmax)'),
    dequantizePerToken: f('int b200q_dequantize_per_token(void *ctx, const void *q, const void *scales, int64_t M, int64_t K, void *y)'),
    quantizeStatic: f('int b200q_quantize_static(void *ctx, const void *x, int64_t n, double scale, int zero_point, int dst_kind, void *q)'),
    dequantizeStatic: f('int b200q_dequantize_static(void *ctx, const void *q, int src_kind, int64_t n, double scale, int zero_point, void *y)'),
    transposeI8: f('int b200q_transpose_i8(void *ctx, const void *w_kn, int64_t K, int64_t N, void *w_nk)'),
    gemmI32: f('int b200q_int8_gemm_i32(void *ctx, const void *A, const void *W, int64_t M, int64_t N, int64_t K, int zpA, int zpW, void *C)'),
    linear: f('int b200q_int8_linear(void *ctx, const void *A, const void *a_scales, const void *W, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out)'),
    linearRequantStatic: f('int b200q_int8_linear_requant_static(void *ctx, const void *A, const void *a_scales, const void *W, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, double out_scale, void *out_q)'),
    linearF32: f('int b200q_linear_f32(void *ctx, const void *x, const void *W, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out)'),
    linearF32Host: f('int b200q_linear_f32_host(void *ctx, const void *x_host, const void *W, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out_host)'),
    linearRequantToken: f('int b200q_int8_linear_requant_token(void *ctx, const void *A, const void *a_scales, const void *W, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out_q, void *out_scales)'),
    quantizeWeightsPerChannel: f('int b200q_quantize_weights_per_channel(void *ctx, const void *w, int64_t N, int64_t K, int layout, void *qw, void *scales32, void *scales64)'),
    setTailMode: f('int b200q_set_tail_mode(void *ctx, int mode)'),
    // calibration on the device (min/max mode)
    observerReset: f('int b200q_observer_reset(void *ctx, void *state)'),
    observeMinmax: f('int b200q_observe_minmax(void *ctx, const void *x, int64_t n, void *state)'),
    // f32 pieces of a transformer block
    embeddingF32: f('int b200q_embedding_f32(void *ctx, const void *table, const void *tokens, const void *pos_table, int64_t M, int64_t D, int64_t V, int64_t S, void *out)'),
    addF32: f('int b200q_add_f32(void *ctx, const void *a, const void *b, int64_t n, void *out)'),
    layernormQuantize: f('int b200q_layernorm_quantize(void *ctx, const void *x, const void *residual, const void *gamma, const void *beta, float eps, int64_t M, int64_t D, void *sum_out, void *y_out, void *q_out, void *scales_out)'),
    sdpaF32: f('int b200q_sdpa_f32(void *ctx, const void *q, const void *k, const void *v, int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t B, int64_t H, int64_t S, int64_t head_dim, float scale, int causal, void *out, int64_t ld_out)'),
  };
}

export function loadB200Q(path: string): B200QBinding {
  if (cached && cached.path === path) return cached.binding;
  cached = { path, binding: bind(path) };
  return cached.binding;
}

/** Turns a non-zero return code into an exception carrying the library's own message. */
export function check(b: B200QBinding, code: number, what: string): void {
  if (code !== 0) throw new Error(`${what}: ${b.lastError() || 'error'} (code ${code})`);
}
