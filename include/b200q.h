/* b200q — C ABI of the B200 backend for mlfw's int8 quantized-inference path.
 *
 * The library is what the TypeScript host of mlfw binds through koffi (the way
 * src/runtime/node/terac.ts:88-101 binds the terac C API).  Conventions follow
 * terac/include/Tera/CAPI/Execution.h:40-81: opaque handle, functions return
 * int (0 = ok) and leave a message for b200q_last_error() otherwise, no
 * exceptions or callbacks cross the boundary, the caller frees what it
 * allocated.
 *
 * Unless a function says "host", every data pointer is a DEVICE pointer obtained
 * from b200q_alloc (or any CUDA allocation on the context's device).  Work is
 * enqueued on the context's stream; b200q_sync waits for it.  A context belongs
 * to one GPU and is not thread safe; distinct contexts may be used concurrently.
 * There is no CPU fallback: without a usable CUDA device b200q_create fails.
 *
 * Paths cited below are inside the reference project (slexisvn/mlfw v0.1.6).
 */
#ifndef B200Q_H
#define B200Q_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b200q_ctx b200q_ctx;

/* Activations of the fused tail (src/compiler/passes/decompose/decomposition_pass.ts:197-230;
 * relu: src/compiler/ir/graph/builder.ts:561-565).  GELU_TANH has no counterpart
 * in the reference (its gelu is the sigmoid form). */
enum { B200Q_ACT_NONE = 0, B200Q_ACT_RELU = 1, B200Q_ACT_GELU_SIGMOID = 2, B200Q_ACT_GELU_TANH = 3, B200Q_ACT_SILU = 4 };
/* Weight layouts: quantized_dot contracts rhs dim 1 ([N,K], a traced Linear) or
 * dim 0 ([K,N]) (src/compiler/ir/graph/ops/quantization.ts:103-154). */
enum { B200Q_W_NK = 0, B200Q_W_KN = 1 };
/* Element kinds of the compiled quantize / dequantize ops (src/compiler/passes/lowering/quant_math.ts:7-14). */
enum { B200Q_I8 = 0, B200Q_UI8 = 1, B200Q_I32 = 2 };

/* ------------------------------------------------------------------ lifetime
 * Replaces device bring-up of the reference CUDA runtime
 * (src/runtime/node/cuda/device.ts:21-32, runtime_api.ts:16-18). */
int b200q_device_count(void);
int b200q_create(int device, b200q_ctx** out);
void b200q_destroy(b200q_ctx* ctx);
const char* b200q_last_error(void);           /* teraLastError, Execution.h:58 */
int b200q_sync(b200q_ctx* ctx);
/* Bits set by kernels that gave up a bounded wait (0 = healthy); reading clears nothing. */
int b200q_status_word(b200q_ctx* ctx, uint32_t* out);
int b200q_clear_status(b200q_ctx* ctx);
/* Bound, in seconds, of every device-side wait of the tensor-core kernel (default 2). */
int b200q_set_wait_limit(b200q_ctx* ctx, double seconds);
/* 0: tensor-core GEMM whenever the shape allows, one CTA or a CTA pair per tile chosen by size (default);
 * 1: CUDA-core kernel only; 2: tensor cores, one CTA per tile; 3: tensor cores, CTA pairs. */
int b200q_set_gemm_variant(b200q_ctx* ctx, int variant);
/* Sigmoid-based tails (gelu_sigmoid, silu) of the tensor-core kernel when the output is f32.
 * 0 (default): every operation rounded as the reference's CPU target rounds it -- bit-identical results, but the exp
 * runs in binary64 and makes those tails about 1.7x longer than the others;
 * 1: hardware exponential and reciprocal -- results within about 1e-6 (relative) of mode 0, inside the 1e-5 bar, at the
 * speed of the other tails.  int8 (requantized) outputs always use the exact form: their codes are integer results. */
int b200q_set_tail_mode(b200q_ctx* ctx, int mode);
/* Epilogue warps of the tensor-core GEMM when the output is f32: 0 (default) = sixteen for the exact sigmoid tails
 * (gelu_sigmoid, silu) when the contraction is short (K <= 1024: the tail, not the tensor pipe, sets the pace there),
 * eight otherwise; 8 or 16 = always that many.  Same results either way. */
int b200q_set_epilogue_warps(b200q_ctx* ctx, int warps);
/* Order in which the tensor-core GEMM's persistent CTAs walk the 256-row x 256-column tiles: -1 (default) = chosen by
 * size (grouped when the weights exceed 48 MB, so that the tiles in flight share W tiles out of L2 instead of streaming
 * all of W from HBM once per row block), 0 = row block by row block, g > 0 = groups of g row blocks.  Same results. */
int b200q_set_tile_group(b200q_ctx* ctx, int row_blocks);
/* Host threads (the caller's included) that stage pageable arrays of the host-buffer entry points through page-locked
 * memory: 0 (default) = half the host's cores, at most 8; takes effect before the first such call of the context. */
int b200q_set_host_threads(b200q_ctx* ctx, int threads);
/* b200q_int8_linear_requant_token and the column-sharded group call: 0 (default) = the GEMM's epilogue publishes every
 * output row's range while the values are in its registers and a one-pass kernel turns the f32 result into codes;
 * 1 = the f32 result goes through the complete per-token quantize (range pass + encode).  Same codes. */
int b200q_set_requant_variant(b200q_ctx* ctx, int variant);
/* Per-token quantize: 0 = rows staged through shared memory by bulk copies when they fit; rows of 8, 12 and 16 KB are
 * moved on into registers and their slot is handed back before the arithmetic (default);
 * 1 = unstaged kernel only; 2 = staged, both passes read shared memory whatever the row length. */
int b200q_set_quant_variant(b200q_ctx* ctx, int variant);
/* Kernels launched through this context since it was created. */
uint64_t b200q_launch_count(b200q_ctx* ctx);
int b200q_sm_count(b200q_ctx* ctx);

/* -------------------------------------------------------------------- memory
 * teraDeviceAlloc / Free / Upload / Download (Execution.h:62-81); the reference
 * CUDA runtime's pool (src/runtime/node/cuda/memory.ts). */
int b200q_alloc(b200q_ctx* ctx, size_t bytes, void** dev);
int b200q_free(b200q_ctx* ctx, void* dev);
int b200q_memset(b200q_ctx* ctx, void* dev, int byte_value, size_t bytes);
int b200q_upload(b200q_ctx* ctx, void* dev, const void* host, size_t bytes);     /* synchronous */
int b200q_download(b200q_ctx* ctx, void* host, const void* dev, size_t bytes);   /* synchronous */
int b200q_host_alloc(b200q_ctx* ctx, size_t bytes, void** host);                 /* page-locked host memory */
int b200q_host_free(b200q_ctx* ctx, void* host);
/* Page-locks an array the caller already holds (a typed array's backing store, src/tensor/core/storage.ts) for as long as
 * it stays registered: the host-buffer entry points then hand it to the copy engines as it is instead of staging it
 * through their own page-locked ring.  Worth it for buffers that are reused over many calls (registering costs about as
 * much as a few calls); unregister before the memory is released. */
int b200q_host_register(b200q_ctx* ctx, void* host, size_t bytes);
int b200q_host_unregister(b200q_ctx* ctx, void* host);

/* -------------------------------------------------------------------- timing
 * CUDA events on the context's stream (the reference times with a host clock:
 * measureCudaKernel, src/runtime/node/cuda_runtime.ts:46-76). */
int b200q_timer_start(b200q_ctx* ctx);
int b200q_timer_stop(b200q_ctx* ctx, float* elapsed_ms);                         /* synchronises */

/* Per-kernel timing: while enabled, every kernel launch is bracketed by CUDA events
 * and its duration added to the sum of its family.  Families (the `kind` argument):
 * 0 quantize_per_token, 1 dequantize_per_token, 2 quantize_static, 3 dequantize_static,
 * 4 weight preparation, 5 tensor-core GEMM (+ fused tail), 6 CUDA-core GEMM, 7 separate tail, 8 embedding,
 * 9 LayerNorm + quantize, 10 attention, 11 residual add.  While profiling is on, the events sit between the kernels, so
 * the dependent launches that let one kernel's set-up overlap the previous kernel's tail are switched off.
 * (No counterpart in the reference, whose runtime only offers measureCudaKernel.) */
int b200q_profile_enable(b200q_ctx* ctx, int on);
int b200q_profile_reset(b200q_ctx* ctx);
int b200q_profile_read(b200q_ctx* ctx, int kind, double* total_ms, uint64_t* launches);   /* synchronises */

/* ------------------------------------------------- per-token (dynamic) ops
 * QuantizationParams.fromConstantArrayPerChannel(x, [M,K], axis 0) +
 * quantizeArrayPerChannel (src/compiler/ir/graph/quantization_types.ts:299-317,118-130):
 * one symmetric scale per row, scale = absMax/127 (row range widened by +-0.5
 * when all entries are equal, non-finite ends replaced by -+1), codes
 * clamp(round_half_up(x / scale)) computed in binary64; NaN stores as 0.
 * scales[m] receives the scale rounded to binary32. */
int b200q_quantize_per_token(b200q_ctx* ctx, const float* x, int64_t M, int64_t K, int8_t* q, float* scales, int qmin,
                             int qmax);
/* dequantizeArrayPerChannel (quantization_types.ts:132-141) with the binary32 scales: y = fround(q * scale[m]). */
int b200q_dequantize_per_token(b200q_ctx* ctx, const int8_t* q, const float* scales, int64_t M, int64_t K, float* y);

/* The same quantization in two steps, for rows whose columns are spread over several GPUs (column-sharded
 * layers; the reference has no multi-device execution): the NaN-ignoring min and max of each row of the local
 * columns, then - after the host has combined them over the GPUs (min of mins, max of maxes) - the codes
 * and the scale from the agreed range.  ld* are row strides in elements.  The codes equal those of
 * b200q_quantize_per_token on the whole row. */
int b200q_row_range(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld, float* row_min, float* row_max);
int b200q_quantize_rows_with_range(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld_in, const float* row_min,
                                   const float* row_max, int8_t* q, int64_t ld_out, float* scales, int qmin, int qmax);

/* ------------------------------------------------- static (compiled) ops
 * The `quantize` / `dequantize` graph ops (src/compiler/ir/graph/ops/quantization.ts:12-101,
 * lowering src/compiler/passes/lowering/rules/quantization.ts:6-21, leaf math quant_math.ts:16-34)
 * exactly as the CPU target evaluates them: fround(x / scale) [+ zero_point], Math.round,
 * clamp to the dtype range, (v|0).  dst_kind: B200Q_I8 or B200Q_UI8. */
int b200q_quantize_static(b200q_ctx* ctx, const float* x, int64_t n, double scale, int zero_point, int dst_kind, void* q);
/* src_kind: B200Q_I8, B200Q_UI8 or B200Q_I32 (the result of quantized_dot). */
int b200q_dequantize_static(b200q_ctx* ctx, const void* q, int src_kind, int64_t n, double scale, int zero_point, float* y);

/* ------------------------------------------------- weights (once per model)
 * QuantizationPass._replacePerChannelDot (src/compiler/passes/quantization/quantization_pass.ts:390-400):
 * per-output-channel symmetric scales and codes of an f32 weight given as [N,K]
 * (B200Q_W_NK) or [K,N] (B200Q_W_KN).  Codes are written K-major, qw[N,K].
 * w_scales64 (binary64, as the pass keeps them) may be null. */
int b200q_quantize_weights_per_channel(b200q_ctx* ctx, const float* w, int64_t N, int64_t K, int layout, int8_t* qw,
                                       float* w_scales32, double* w_scales64);
/* Per-group symmetric quantization of a constant (GPTQ / AWQ-style INT4): QuantizationParams.fromConstantArrayPerGroup
 * and quantizeArrayPerGroup (src/compiler/ir/graph/quantization_types.ts:319-340, 143-153).  Groups are runs of
 * group_size consecutive elements of the flat array x[n] (the last may be shorter); scale = absMax / (2^(bits-1) - 1),
 * or 1e-10 when that is 0, in binary64; codes = clamp(Math.round(x / scale)) to [-2^(bits-1), 2^(bits-1) - 1], one per
 * int8 as the reference keeps them (not packed).  num_bits 2..8.  q, scales64, scales32 may each be null. */
int b200q_quantize_per_group(b200q_ctx* ctx, const float* x, int64_t n, int64_t group_size, int num_bits, int8_t* q,
                             double* scales64, float* scales32);
/* dequantizeArrayPerGroup (quantization_types.ts:155-162): (q - 0) * scale[group] in binary64; y32 is that number
 * stored to a Float32Array.  Either output may be null. */
int b200q_dequantize_per_group(b200q_ctx* ctx, const int8_t* q, int64_t n, int64_t group_size, const double* scales64,
                               double* y64, float* y32);
/* Re-lay int8 weights [K,N] as [N,K] (the layout the tensor-core kernel reads). */
int b200q_transpose_i8(b200q_ctx* ctx, const int8_t* w_kn, int64_t K, int64_t N, int8_t* w_nk);

/* ------------------------------------------------- contraction and tail
 * quantized_dot (ops/quantization.ts:103-154; lowering rules/quantization.ts:23-42):
 * C[m,n] = sum_k (A[m,k]-zpA) * (W[n,k]-zpW), int32.  W is [N,K].  Tensor cores when K is a multiple of 16 and the
 * operands are 16-byte aligned -- with zero-points as the plain product plus the three correction terms
 * (-zpW * sum_k A, -zpA * sum_k W, K * zpA * zpW; two row-sum launches and one pass over C) -- the CUDA cores otherwise. */
int b200q_int8_gemm_i32(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K, int zpA,
                        int zpW, int32_t* C);
/* quantized_conv with two spatial dimensions (ops/quantization.ts:156-190; lowering rules/quantization.ts:44-62 over
 * the loop nest of src/compiler/passes/lowering/lowering_registry.ts:335-449; extents ops/linalg.ts:236-246):
 *   out[n,oc,oh,ow] = sum_{ic,kh,kw} (in[n, g*C/groups + ic, oh*sh + kh*dh - pad_top, ow*sw + kw*dw - pad_left] - zp_in)
 *                                    * (ker[oc,ic,kh,kw] - zp_ker),   g = oc / (O / groups),
 * a tap outside the input adds 0; int32.  layout B200Q_CONV_NCHW: input [N,C,H,W], kernel [O,C/groups,KH,KW], output
 * [N,O,OH,OW] (the reference's); B200Q_CONV_NHWC: input [N,H,W,C], kernel [O,KH,KW,C/groups], output [N,OH,OW,O].
 * Runs as gather + contraction (tensor cores when both zero-points are 0) through context-owned workspaces of
 * N*OH*OW*ceil16(C/groups*KH*KW) bytes and, unless the output is channel-last with one group, 4*N*OH*OW*O/groups;
 * a channel-first call with a multiple of 16 channels per group also re-lays input and kernel channel-last
 * (N*C*H*W + O*C/groups*KH*KW bytes more).  Channel-last with C/groups a multiple of 16 is the fast form. */
#define B200Q_CONV_NCHW 0
#define B200Q_CONV_NHWC 1
int b200q_quantized_conv2d(b200q_ctx* ctx, const int8_t* in, const int8_t* ker, int64_t N, int64_t C, int64_t H, int64_t W,
                           int64_t O, int64_t KH, int64_t KW, int stride_h, int stride_w, int pad_top, int pad_bottom,
                           int pad_left, int pad_right, int dil_h, int dil_w, int groups, int zp_in, int zp_ker, int layout,
                           int32_t* out);
/* ui8 operands of quantized_dot / quantized_conv (QUANTIZED_INT_DTYPES, ops/quantization.ts:8,146-151): dst[i] = src[i] - 128
 * as int8 (src may equal dst).  u - zp == (u - 128) - (zp - 128), so the contraction entry points take the shifted
 * codes with the zero-point moved by 128 and give the reference's sums. */
int b200q_shift_u8_to_i8(b200q_ctx* ctx, const uint8_t* src, int64_t n, int8_t* dst);
/* The per-channel tail as separate ops (quantization_pass.ts:427-456, nn/functional/linear.ts:13-15):
 * out = act(fround(fround(acc * sv) + bias[n])) with sv = fround(a_scales[m] * w_scales[n]),
 * or sv = w_scales[n] when a_scales is null (static activation scale folded by the host). */
int b200q_epilogue(b200q_ctx* ctx, const int32_t* acc, int64_t M, int64_t N, const float* a_scales, const float* w_scales,
                   const float* bias, int act, float* out);
/* The per-tensor tail (quantization_pass.ts:286-360): `dequantize{scale}` of the int32 sums -- fround((double)acc * scale)
 * with the scale a binary64 immediate, as the compiled op evaluates it (quant_math.ts:29-34) -- then the same optional
 * bias and activation. */
int b200q_epilogue_tensor_scale(b200q_ctx* ctx, const int32_t* acc, int64_t M, int64_t N, double scale, const float* bias,
                                int act, float* out);
/* quantized_dot + tail in one kernel.  A int8 [M,K], W int8 [N,K]. */
int b200q_int8_linear(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W_nk, const float* w_scales,
                      const float* bias, int act, int64_t M, int64_t N, int64_t K, float* out);
/* b200q_int8_linear for activations stored as `a_blocks` equal column blocks, block r an int8 row-major
 * [M, K / a_blocks] matrix at A + r * M * (K / a_blocks): what an all-gather of column-sharded activations leaves
 * (see b200q_group_linear_nshard; no counterpart in the reference).  The kernel reads the blocks in place through a
 * three-dimensional tensor map.  K / a_blocks must be a multiple of 128; tensor-core shapes only. */
int b200q_int8_linear_gathered(b200q_ctx* ctx, const int8_t* A, const float* a_scales, int a_blocks, const int8_t* W_nk,
                               const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K, float* out);
/* Same, followed by the next layer's static `quantize` (scale out_scale, zero-point 0, int8) inside the epilogue. */
int b200q_int8_linear_requant_static(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W_nk,
                                     const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K,
                                     double out_scale, int8_t* out_q);
/* Same, followed by the next layer's per-token quantize (two kernels: the f32 result
 * goes through a context-owned workspace). */
int b200q_int8_linear_requant_token(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W_nk,
                                    const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K,
                                    int8_t* out_q, float* out_scales);
/* Same, with the f32 result kept as well (out_f32 [M,N], e.g. for a residual branch) instead of a workspace. */
int b200q_int8_linear_f32_requant_token(b200q_ctx* ctx, const int8_t* A, const float* a_scales, const int8_t* W_nk,
                                        const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K,
                                        float* out_f32, int8_t* out_q, float* out_scales);
/* The whole hot path from f32 activations: per-token quantize (into a context-owned
 * workspace), contraction, tail. */
int b200q_linear_f32(b200q_ctx* ctx, const float* x, const int8_t* W_nk, const float* w_scales, const float* bias, int act,
                     int64_t M, int64_t N, int64_t K, float* out);
/* b200q_linear_f32 for callers that must not allocate device memory inside the call (a host whose own pool
 * owns the device, a latency-bound serving loop, a phase in which the CUDA allocation calls are not allowed).
 * This entry point has no counterpart in the reference.  Same arguments and result as b200q_linear_f32; the
 * int8 codes and per-token scales of the activations go to a fixed array of static device memory inside the
 * library instead of a workspace, so: M * K <= 4 Mi elements and M <= 16384 rows, and the shape must be one the
 * tensor-core kernel takes (K a multiple of 16, 16-byte aligned weights) - anything else is rejected with an error.
 * The array (4 MiB + 64 KiB) exists on every device on which this process has created a context with
 * b200q_create - that call loads the array's module on the device and looks its address up, so the memory is
 * reserved at context creation, not in here - and lives until that device's CUDA context is destroyed (normally
 * process exit); devices the process never creates a context on hold nothing.  It is shared by all calls on a
 * device and keeps the last call's contents (nothing in it needs to start at zero).  Calls on one context may be
 * enqueued back to back; calls that overlap on one device (two contexts, two host threads) race on the array.
 * The entry point calls no CUDA allocation routine.  The CUDA runtime still loads a kernel's code on its first
 * launch and this library sets a per-kernel attribute on first use, so a host that must have even that out of the
 * way (before handing all device memory to its pool, or before a stream capture) makes one warm-up call per
 * activation and shape class (M below / from 1024 rows; row length 8, 12, 16 KB or other) it is going to use. */
int b200q_linear_f32_noalloc(b200q_ctx* ctx, const float* x, const int8_t* W_nk, const float* w_scales, const float* bias,
                             int act, int64_t M, int64_t N, int64_t K, float* out);
/* `count` independent batches x[i] [M,K] -> out[i] [M,N] through the same weights (a serving loop's queue; no
 * counterpart in the reference, whose compiled function takes one batch per call): the per-token quantize of batch i+1
 * runs on a second stream of the context while the GEMM of batch i holds the tensor cores.  Results are those of
 * b200q_linear_f32, batch by batch.  x and out are host arrays of device pointers.  Stream-ordered like every call. */
int b200q_linear_f32_many(b200q_ctx* ctx, int count, const float* const* x, const int8_t* W_nk, const float* w_scales,
                          const float* bias, int act, int64_t M, int64_t N, int64_t K, float* const* out);
/* Same call with HOST activations and HOST result (what RuntimeModule.run hands a
 * backend: typed arrays, src/runtime/runtime.ts:239-268); weights stay on the device.
 * Copies both ways and synchronises.  Row blocks are pipelined: one on its way in, one computing, one on its way out.
 * Page-locked (cudaHostAlloc / cudaHostRegister) arrays go to the copy engines as they are; ordinary (pageable) arrays
 * -- what a caller holding typed arrays has -- are staged block by block through a page-locked ring of the context
 * (3 blocks per direction, allocated at the first such call) by a few host threads of the context. */
int b200q_linear_f32_host(b200q_ctx* ctx, const float* x_host, const int8_t* W_nk, const float* w_scales, const float* bias,
                          int act, int64_t M, int64_t N, int64_t K, float* out_host);
/* Host-buffer round trip of the standalone ops: quantize_per_token then dequantize_per_token. */
int b200q_quant_roundtrip_host(b200q_ctx* ctx, const float* x_host, int64_t M, int64_t K, int8_t* q_host, float* scales_host,
                               float* y_host);

/* ---- calibration on the device (min/max mode) ----
 * A calibration observer keeps the running minimum and maximum of every value of an observed tensor, NaN ignored
 * (ValueObserver.update, src/compiler/analysis/calibration.ts:24-30).  `state` is two floats of device memory:
 * state[0] = min, state[1] = max; b200q_observer_reset sets them to +Inf / -Inf ("nothing seen").  The quantization
 * parameters follow on the host from QuantizationParams.fromRange (quantization_types.ts:248-263). */
int b200q_observer_reset(b200q_ctx* ctx, float* state);
int b200q_observe_minmax(b200q_ctx* ctx, const float* x, int64_t n, float* state);

/* Histogram modes of the calibration observer (percentile 0.999 and entropy; HistogramCollector,
 * src/compiler/analysis/calibration.ts:41-186).  b200q_histogram_f32 adds the n values of x to `bins` (num_bins 64-bit
 * counters in device memory, at most 4096) exactly as HistogramCollector.update bins them: index
 * min(num_bins - 1, floor((v - range_min) * (num_bins / (range_max - range_min)))) in binary64; NaN lands in no bin;
 * nothing is counted when the range is empty.  The caller keeps the range covering the data (the reference widens it
 * and re-buckets on the host when a batch falls outside: mlfw_b200/calibration.py does the same with 2048 numbers).
 * The two threshold functions are HOST arithmetic on the downloaded counts (bins as binary64, like the reference's
 * Float64Array) and need no device: computePercentileThreshold (:130-141) and computeEntropyThreshold (:143-186),
 * the sums taken in the reference's order. */
int b200q_histogram_f32(b200q_ctx* ctx, const float* x, int64_t n, double range_min, double range_max, int num_bins,
                        uint64_t* bins);
int b200q_histogram_percentile_threshold(const double* bins, int num_bins, double total_count, double range_min, double range_max,
                                         double percentile, double* threshold);
int b200q_histogram_entropy_threshold(const double* bins, int num_bins, double total_count, double range_min, double range_max,
                                      int num_quant_bins, double* threshold);

/* ---- f32 pieces of a transformer block around the int8 linears ("next" components of the hot path) ----
 * Floating-point kernels: results agree with the reference's CPU target to 1e-5 of the output's largest magnitude
 * (its own summation order depends on which lowering runs); the int8 codes b200q_layernorm_quantize emits are the exact
 * per-token quantization of the binary32 values it would store as y_out. */

/* out[m, :] = table[tokens[m], :] (+ pos_table[m % S, :] when pos_table is not null).  table f32 [V, D], tokens int32 [M],
 * pos_table f32 [S, D], out f32 [M, D]; D a multiple of 4.  src/nn/functional/embedding.ts:6-11; positions as in
 * tests/_utils/gpt2_model.js:11-13.  A token outside [0, V) gives a zero row and sets a status bit. */
int b200q_embedding_f32(b200q_ctx* ctx, const float* table, const int32_t* tokens, const float* pos_table, int64_t M, int64_t D,
                        int64_t V, int64_t S, float* out);
/* out = a + b elementwise (one rounding per element: ops.add), n a multiple of 4.  src/nn/modules/transformer.ts:144-152. */
int b200q_add_f32(b200q_ctx* ctx, const float* a, const float* b, int64_t n, float* out);
/* LayerNorm over the last axis of x [M, D] (+ residual [M, D] first, when given), then per-token int8 quantization of
 * the result for the linear that follows.  gamma, beta f32 [D]; D a multiple of 4, at most 2048.  Outputs, each
 * optional (null): sum_out = x + residual [M, D]; y_out = the normalised rows f32 [M, D]; q_out int8 [M, D] with
 * scales_out f32 [M].  src/compiler/passes/decompose/decomposition_pass.ts:232-260 followed by
 * src/compiler/ir/graph/quantization_types.ts:299-317, 118-130 along axis 0. */
int b200q_layernorm_quantize(b200q_ctx* ctx, const float* x, const float* residual, const float* gamma, const float* beta,
                             float eps, int64_t M, int64_t D, float* sum_out, float* y_out, int8_t* q_out, float* scales_out);
/* softmax(q k^T * scale + mask) v per (batch, head) in binary32; head dimension 64.  Row (b, s) of head h starts at
 * base + (b*S + s)*ld + h*64 for q, k, v and out (so the projections are read where the linears wrote them);
 * causal != 0 masks keys j > i.  src/nn/functional/attention.ts:42-74. */
/* Which kernel b200q_sdpa_f32 runs.  0 (default): the tensor-core kernel (tcgen05.mma.kind::tf32 with every product
 * taken three ways - hi*hi + hi*lo + lo*hi - so the result keeps binary32 accuracy, scores and P in tensor memory)
 * whenever the buffers are 16-byte aligned; otherwise the CUDA-core kernel.  1: warp-level mma.sync with the same
 * three-way products.  2: the tensor-core kernel or an error.  3: CUDA cores, binary32 FMA.  All meet the 1e-5 bar. */
int b200q_set_sdpa_variant(b200q_ctx* ctx, int variant);
int b200q_sdpa_f32(b200q_ctx* ctx, const float* q, const float* k, const float* v, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                   int64_t B, int64_t H, int64_t S, int64_t head_dim, float scale, int causal, float* out, int64_t ld_out);

/* ---- captured steps ----
 * A sequence of calls on a context recorded once and replayed with one launch (the reference's CUDA runtime replays
 * captured plans and eager steps the same way: src/runtime/node/cuda/eager_graph.ts:16-41, device_plan.ts:178-219).
 * Between begin and end every call on the context is recorded instead of executed; calls that synchronise or copy to
 * or from host memory are not allowed there, and every workspace must already have its size: run the same calls once,
 * not captured, before capturing them.  The recorded pointers and shapes are fixed; replay as often as wanted. */
typedef struct b200q_graph b200q_graph;
int b200q_graph_begin(b200q_ctx* ctx);
int b200q_graph_end(b200q_ctx* ctx, b200q_graph** out);
int b200q_graph_launch(b200q_ctx* ctx, b200q_graph* graph);
int b200q_graph_destroy(b200q_ctx* ctx, b200q_graph* graph);

/* ---- self test of the bounded device-side wait ----
 * Launches one thread that waits, with the library's own wait routine and the given limit (seconds, at most 1), on a
 * barrier in its shared memory that nothing ever signals, with no asynchronous work in flight.  The wait must give up:
 * the kernel then sets bit 6 of the status word and returns.  For tests of the give-up path on a healthy device. */
int b200q_selftest_bounded_wait(b200q_ctx* ctx, double limit_seconds);

/* ---- several GPUs of one node ----
 * The reference executes on one device (src/runtime/node/cuda/runtime_api.ts:16-18); nothing below has a counterpart
 * there.  A group is one NCCL communicator with one rank per GPU.  Either one process drives several of its GPUs
 * (b200q_group_create: the group creates and owns one context per device, rank i = devices[i]) or every GPU has its
 * own process (b200q_group_create_rank: the process passes its context; the 128-byte id comes from
 * b200q_group_unique_id on one rank and reaches the others by the host's own means).  The per-GPU arguments of the
 * calls below are arrays with one entry per LOCAL rank (b200q_group_local_count: n, or 1), holding device pointers
 * on that rank's GPU.  NCCL is loaded when the first group function is called: the libnccl.so.2 the process already
 * holds if there is one, else the file named by the environment variable B200Q_NCCL_LIBRARY, else the system's.  Two
 * different NCCL builds do not mix in one process, so a host that brings its own loads it first. */
typedef struct b200q_group b200q_group;
int b200q_group_unique_id(void* id128);                       /* host buffer of 128 bytes */
int b200q_group_create(const int* devices, int n, b200q_group** out);
int b200q_group_create_rank(b200q_ctx* ctx, const void* id128, int rank, int world, b200q_group** out);
int b200q_group_destroy(b200q_group* group);
int b200q_group_world(b200q_group* group);                    /* ranks of the communicator */
int b200q_group_local_count(b200q_group* group);              /* ranks this process drives */
b200q_ctx* b200q_group_ctx(b200q_group* group, int local_index);
int b200q_group_rank(b200q_group* group, int local_index);
int b200q_group_nccl_version(b200q_group* group, int* version);
/* Waits (host) for everything queued on the local ranks' streams. */
int b200q_group_sync(b200q_group* group);
/* Rows sharded: local rank i computes b200q_linear_f32 on its own rows[i] rows against its replica of the weights.
 * No collective: a row depends on nothing but itself. */
int b200q_group_linear_mshard(b200q_group* group, const float* const* x, const int64_t* rows, const int8_t* const* W_nk,
                              const float* const* w_scales, const float* const* bias, int act, int64_t N, int64_t K,
                              float* const* out);
/* Output channels sharded: every rank holds the int8 activations of all M rows (q_in, in_scales [M]) and the weights,
 * scales and bias of its own N / world channels (W_shard int8 [N/world, K], rank r owns channels [r*N/world, ...)).
 * Either out_f32 is given: local rank i receives its channels of the result, f32 [M, N/world] - no collective; or
 * q_out and out_scales are given: the result is requantized per token exactly as one GPU would (the rows' ranges are
 * agreed by one max-reduction over the ranks) and the int8 column blocks are all-gathered, so that every rank ends
 * up with all codes and scales [M].  The gathered codes are left in the layout the all-gather produces - per row
 * chunk (see b200q_group_set_chunks; one chunk by default), the ranks' blocks one after the other, block r an int8
 * [rows of the chunk, N/world] matrix; chunk c starts at q_out + N * (first row of the chunk) - and the next call
 * takes them as they are with in_blocks = world (in_blocks = 1: q_in is an ordinary row-major [M, K] matrix).
 * N must divide by world, and N/world by 128 for a gathered output.  bias may be null (the array or its entries). */
int b200q_group_linear_nshard(b200q_group* group, const int8_t* const* q_in, const float* const* in_scales, int in_blocks,
                              const int8_t* const* W_shard, const float* const* w_scales, const float* const* bias, int act,
                              int64_t M, int64_t N, int64_t K, int8_t* const* q_out, float* const* out_scales,
                              float* const* out_f32);
/* Row chunks of the column-sharded call (default 1).  With more than one, the collectives of a chunk run on a second
 * stream while the next chunk's GEMM computes, and a following column-sharded call starts on its first chunk while
 * later chunks are still being gathered; chunks are whole multiples of 256 rows.  After a chunked call the gathered
 * output is complete on the contexts' streams only once b200q_group_fence (or _sync, or the next column-sharded call,
 * chunk by chunk) has been issued. */
int b200q_group_set_chunks(b200q_group* group, int chunks);
int b200q_group_fence(b200q_group* group);
/* All-gather of `bytes` bytes per rank on the contexts' streams: recv[i] receives world * bytes, rank after rank. */
int b200q_group_all_gather(b200q_group* group, const void* const* send, void* const* recv, size_t bytes);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H */
