// koffi binding of libb200q.so — the C ABI declared in include/b200q.h.
// Same idiom as the reference's terac binding (src/runtime/node/terac.ts:88-101):
// koffi.load + lib.func('<C prototype>'), one cached binding per library path.
// One entry per declaration of the header, in the header's order; tests/test_ts_binding.py parses the prototype
// strings below and holds them to include/b200q.h (names, argument counts, scalar types).
// This file is source only in this repository: no JavaScript engine exists in the
// build image, so it is exercised through its Python twin (mlfw_b200/_lib.py).
// Pointer arguments: device and host buffers are `void *`; `void **` is an array with one device pointer per local
// rank of a group (koffi takes a JavaScript array of pointers); `_Out_` marks values the call writes for the caller.
import koffi from 'koffi';

export type B200QBinding = ReturnType<typeof bind>;

let cached: { path: string; binding: B200QBinding } | null = null;

function bind(path: string) {
  const lib = koffi.load(path);
  const f = (proto: string) => lib.func(proto);
  return {
    deviceCount: f('int b200q_device_count()'),
    create: f('int b200q_create(int device, _Out_ void **out)'),
    destroy: f('void b200q_destroy(void *ctx)'),
    lastError: f('str b200q_last_error()'),
    sync: f('int b200q_sync(void *ctx)'),
    statusWord: f('int b200q_status_word(void *ctx, _Out_ uint32_t *out)'),
    clearStatus: f('int b200q_clear_status(void *ctx)'),
    setWaitLimit: f('int b200q_set_wait_limit(void *ctx, double seconds)'),
    setGemmVariant: f('int b200q_set_gemm_variant(void *ctx, int variant)'),
    setTailMode: f('int b200q_set_tail_mode(void *ctx, int mode)'),
    setEpilogueWarps: f('int b200q_set_epilogue_warps(void *ctx, int warps)'),
    setTileGroup: f('int b200q_set_tile_group(void *ctx, int row_blocks)'),
    setHostThreads: f('int b200q_set_host_threads(void *ctx, int threads)'),
    setRequantVariant: f('int b200q_set_requant_variant(void *ctx, int variant)'),
    setQuantVariant: f('int b200q_set_quant_variant(void *ctx, int variant)'),
    launchCount: f('uint64_t b200q_launch_count(void *ctx)'),
    smCount: f('int b200q_sm_count(void *ctx)'),
    alloc: f('int b200q_alloc(void *ctx, size_t bytes, _Out_ void **dev)'),
    free: f('int b200q_free(void *ctx, void *dev)'),
    memset: f('int b200q_memset(void *ctx, void *dev, int byte_value, size_t bytes)'),
    upload: f('int b200q_upload(void *ctx, void *dev, const void *host, size_t bytes)'),
    download: f('int b200q_download(void *ctx, void *host, const void *dev, size_t bytes)'),
    hostAlloc: f('int b200q_host_alloc(void *ctx, size_t bytes, _Out_ void **host)'),
    hostFree: f('int b200q_host_free(void *ctx, void *host)'),
    hostRegister: f('int b200q_host_register(void *ctx, void *host, size_t bytes)'),
    hostUnregister: f('int b200q_host_unregister(void *ctx, void *host)'),
    timerStart: f('int b200q_timer_start(void *ctx)'),
    timerStop: f('int b200q_timer_stop(void *ctx, _Out_ float *elapsed_ms)'),
    profileEnable: f('int b200q_profile_enable(void *ctx, int on)'),
    profileReset: f('int b200q_profile_reset(void *ctx)'),
    profileRead: f('int b200q_profile_read(void *ctx, int kind, _Out_ double *total_ms, _Out_ uint64_t *launches)'),
    quantizePerToken: f('int b200q_quantize_per_token(void *ctx, const void *x, int64_t M, int64_t K, void *q, void *scales, int qmin, int qmax)'),
    dequantizePerToken: f('int b200q_dequantize_per_token(void *ctx, const void *q, const void *scales, int64_t M, int64_t K, void *y)'),
    rowRange: f('int b200q_row_range(void *ctx, const void *y, int64_t M, int64_t N, int64_t ld, void *row_min, void *row_max)'),
    quantizeRowsWithRange: f('int b200q_quantize_rows_with_range(void *ctx, const void *y, int64_t M, int64_t N, int64_t ld_in, const void *row_min, const void *row_max, void *q, int64_t ld_out, void *scales, int qmin, int qmax)'),
    quantizeStatic: f('int b200q_quantize_static(void *ctx, const void *x, int64_t n, double scale, int zero_point, int dst_kind, void *q)'),
    dequantizeStatic: f('int b200q_dequantize_static(void *ctx, const void *q, int src_kind, int64_t n, double scale, int zero_point, void *y)'),
    quantizeWeightsPerChannel: f('int b200q_quantize_weights_per_channel(void *ctx, const void *w, int64_t N, int64_t K, int layout, void *qw, void *w_scales32, void *w_scales64)'),
    quantizePerGroup: f('int b200q_quantize_per_group(void *ctx, const void *x, int64_t n, int64_t group_size, int num_bits, void *q, void *scales64, void *scales32)'),
    dequantizePerGroup: f('int b200q_dequantize_per_group(void *ctx, const void *q, int64_t n, int64_t group_size, const void *scales64, void *y64, void *y32)'),
    transposeI8: f('int b200q_transpose_i8(void *ctx, const void *w_kn, int64_t K, int64_t N, void *w_nk)'),
    int8GemmI32: f('int b200q_int8_gemm_i32(void *ctx, const void *A, const void *W_nk, int64_t M, int64_t N, int64_t K, int zpA, int zpW, void *C)'),
    quantizedConv2d: f('int b200q_quantized_conv2d(void *ctx, const void *in, const void *ker, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O, int64_t KH, int64_t KW, int stride_h, int stride_w, int pad_top, int pad_bottom, int pad_left, int pad_right, int dil_h, int dil_w, int groups, int zp_in, int zp_ker, int layout, void *out)'),
    shiftU8ToI8: f('int b200q_shift_u8_to_i8(void *ctx, const void *src, int64_t n, void *dst)'),
    epilogue: f('int b200q_epilogue(void *ctx, const void *acc, int64_t M, int64_t N, const void *a_scales, const void *w_scales, const void *bias, int act, void *out)'),
    epilogueTensorScale: f('int b200q_epilogue_tensor_scale(void *ctx, const void *acc, int64_t M, int64_t N, double scale, const void *bias, int act, void *out)'),
    int8Linear: f('int b200q_int8_linear(void *ctx, const void *A, const void *a_scales, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out)'),
    int8LinearGathered: f('int b200q_int8_linear_gathered(void *ctx, const void *A, const void *a_scales, int a_blocks, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out)'),
    int8LinearRequantStatic: f('int b200q_int8_linear_requant_static(void *ctx, const void *A, const void *a_scales, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, double out_scale, void *out_q)'),
    int8LinearRequantToken: f('int b200q_int8_linear_requant_token(void *ctx, const void *A, const void *a_scales, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out_q, void *out_scales)'),
    int8LinearF32RequantToken: f('int b200q_int8_linear_f32_requant_token(void *ctx, const void *A, const void *a_scales, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out_f32, void *out_q, void *out_scales)'),
    linearF32: f('int b200q_linear_f32(void *ctx, const void *x, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out)'),
    linearF32Noalloc: f('int b200q_linear_f32_noalloc(void *ctx, const void *x, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out)'),
    linearF32Many: f('int b200q_linear_f32_many(void *ctx, int count, void **x, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void **out)'),
    linearF32Host: f('int b200q_linear_f32_host(void *ctx, const void *x_host, const void *W_nk, const void *w_scales, const void *bias, int act, int64_t M, int64_t N, int64_t K, void *out_host)'),
    quantRoundtripHost: f('int b200q_quant_roundtrip_host(void *ctx, const void *x_host, int64_t M, int64_t K, void *q_host, void *scales_host, void *y_host)'),
    observerReset: f('int b200q_observer_reset(void *ctx, void *state)'),
    observeMinmax: f('int b200q_observe_minmax(void *ctx, const void *x, int64_t n, void *state)'),
    histogramF32: f('int b200q_histogram_f32(void *ctx, const void *x, int64_t n, double range_min, double range_max, int num_bins, void *bins)'),
    histogramPercentileThreshold: f('int b200q_histogram_percentile_threshold(const void *bins, int num_bins, double total_count, double range_min, double range_max, double percentile, _Out_ double *threshold)'),
    histogramEntropyThreshold: f('int b200q_histogram_entropy_threshold(const void *bins, int num_bins, double total_count, double range_min, double range_max, int num_quant_bins, _Out_ double *threshold)'),
    embeddingF32: f('int b200q_embedding_f32(void *ctx, const void *table, const void *tokens, const void *pos_table, int64_t M, int64_t D, int64_t V, int64_t S, void *out)'),
    addF32: f('int b200q_add_f32(void *ctx, const void *a, const void *b, int64_t n, void *out)'),
    layernormQuantize: f('int b200q_layernorm_quantize(void *ctx, const void *x, const void *residual, const void *gamma, const void *beta, float eps, int64_t M, int64_t D, void *sum_out, void *y_out, void *q_out, void *scales_out)'),
    setSdpaVariant: f('int b200q_set_sdpa_variant(void *ctx, int variant)'),
    sdpaF32: f('int b200q_sdpa_f32(void *ctx, const void *q, const void *k, const void *v, int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t B, int64_t H, int64_t S, int64_t head_dim, float scale, int causal, void *out, int64_t ld_out)'),
    graphBegin: f('int b200q_graph_begin(void *ctx)'),
    graphEnd: f('int b200q_graph_end(void *ctx, _Out_ void **out)'),
    graphLaunch: f('int b200q_graph_launch(void *ctx, void *graph)'),
    graphDestroy: f('int b200q_graph_destroy(void *ctx, void *graph)'),
    selftestBoundedWait: f('int b200q_selftest_bounded_wait(void *ctx, double limit_seconds)'),
    groupUniqueId: f('int b200q_group_unique_id(void *id128)'),
    groupCreate: f('int b200q_group_create(const int *devices, int n, _Out_ void **out)'),
    groupCreateRank: f('int b200q_group_create_rank(void *ctx, const void *id128, int rank, int world, _Out_ void **out)'),
    groupDestroy: f('int b200q_group_destroy(void *group)'),
    groupWorld: f('int b200q_group_world(void *group)'),
    groupLocalCount: f('int b200q_group_local_count(void *group)'),
    groupCtx: f('void *b200q_group_ctx(void *group, int local_index)'),
    groupRank: f('int b200q_group_rank(void *group, int local_index)'),
    groupNcclVersion: f('int b200q_group_nccl_version(void *group, _Out_ int *version)'),
    groupSync: f('int b200q_group_sync(void *group)'),
    groupLinearMshard: f('int b200q_group_linear_mshard(void *group, void **x, const int64_t *rows, void **W_nk, void **w_scales, void **bias, int act, int64_t N, int64_t K, void **out)'),
    groupLinearNshard: f('int b200q_group_linear_nshard(void *group, void **q_in, void **in_scales, int in_blocks, void **W_shard, void **w_scales, void **bias, int act, int64_t M, int64_t N, int64_t K, void **q_out, void **out_scales, void **out_f32)'),
    groupSetChunks: f('int b200q_group_set_chunks(void *group, int chunks)'),
    groupFence: f('int b200q_group_fence(void *group)'),
    groupAllGather: f('int b200q_group_all_gather(void *group, void **send, void **recv, size_t bytes)'),
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
