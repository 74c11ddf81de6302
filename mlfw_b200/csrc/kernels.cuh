// Launchers implemented by the kernel translation units; called by the C ABI (api.cu).
// All of them enqueue on ctx->stream and return 0 or a non-zero code after set_error().
#pragma once
#include <cstddef>
#include <cstdint>

struct b200q_ctx;

namespace b200q {

int launch_quantize_per_token(b200q_ctx* ctx, const float* x, int64_t M, int64_t K, int8_t* q, float* scales, int qmin, int qmax);
int launch_dequantize_per_token(b200q_ctx* ctx, const int8_t* q, const float* scales, int64_t M, int64_t K, float* y);
// dst_kind / src_kind: 0 = int8, 1 = uint8, 2 = int32 (source of dequantize only)
int launch_quantize_static(b200q_ctx* ctx, const float* x, int64_t n, double scale, int zp, int dst_kind, void* q);
int launch_dequantize_static(b200q_ctx* ctx, const void* q, int src_kind, int64_t n, double scale, int zp, float* y);
// layout 0: w is [N,K]; 1: w is [K,N].  Codes are always written [N,K].
int launch_quantize_weights(b200q_ctx* ctx, const float* w, int64_t N, int64_t K, int layout, int qmin, int qmax, int8_t* qw,
                            float* scales32, double* scales64);
// Two-step per-token quantize for rows that are spread over several GPUs (column-sharded layers).
// ld / ld_in / ld_out: row strides in elements (a shard may be a column block of a wider buffer).
int launch_row_range(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld, float* mn, float* mx);
int launch_quantize_rows_with_range(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld_in, const float* mn,
                                    const float* mx, int8_t* q, int64_t ld_out, float* scales, int qmin, int qmax);
// The second step of the per-token quantize when the ranges were published as keys by the kernel that produced y
// (keys: [0, M) maxima, [M, 2M) minima; 0 = nothing seen).  One streaming pass: reads y once, writes the codes.
int launch_quantize_rows_with_keys(b200q_ctx* ctx, const float* y, int64_t M, int64_t N, int64_t ld_in, const uint32_t* keys,
                                   int8_t* q, int64_t ld_out, float* scales, int qmin, int qmax);
// keys[0..2M) from separate min / max arrays (the result of launch_row_range), for the CUDA-core path.
int launch_range_to_keys(b200q_ctx* ctx, const float* mn, const float* mx, int64_t M, uint32_t* keys);
int launch_transpose_i8(b200q_ctx* ctx, const int8_t* src_kn, int64_t K, int64_t N, int8_t* dst_nk);
// Adds the values of x to a histogram of num_bins (<= 4096) equal bins over [range_min, range_max] (64-bit counters in device memory).
int launch_histogram_f32(b200q_ctx* ctx, const float* x, int64_t n, double range_min, double range_max, int num_bins,
                         unsigned long long* bins);
// Running min / max of a calibration observer: state[0] = min, state[1] = max (device memory, +Inf / -Inf when new).
int launch_minmax_observe(b200q_ctx* ctx, const float* x, int64_t n, float* state);

int launch_gemm_i8_simt(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K, int zpA, int zpB,
                        int32_t* C);
// dst[i] = (int8)(src[i] - 128): an unsigned operand of a contraction becomes a signed one with its zero-point 128 lower.
int launch_shift_u8_i8(b200q_ctx* ctx, const uint8_t* src, int64_t n, int8_t* dst);
// Turns the plain product sum_k a w in C into sum_k (a - zpA)(w - zpB): row sums of both operands and one pass over C.
// `sums`: M + N words of scratch.
int launch_zero_point_fix(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K, int zpA, int zpB,
                          int32_t* sums, int32_t* C);
// int32 contraction with zero-points by whichever kernel takes the shape: the tensor cores (plus the zero-point
// correction) when the operands are 16-byte aligned and K is a multiple of 16, the CUDA cores otherwise.
int gemm_i32_any(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K, int zpA, int zpB, int32_t* C);
// Exactly one of out_f32 / out_q is written (both may be given); out_q uses the static scale q_scale.
// w_scales == null: one binary64 scale for the whole tensor (tensor_scale), applied as the compiled `dequantize` does.
int launch_epilogue(b200q_ctx* ctx, const int32_t* acc, int64_t M, int64_t N, const float* a_scales, const float* w_scales,
                    const float* bias, int act, float* out_f32, int8_t* out_q, double q_scale, double tensor_scale = 0.0);

bool gemm_umma_supported(const void* A, const void* W, int64_t M, int64_t N, int64_t K);
// Tensor-core GEMM with the fused tail.  out_i32 != null: raw accumulators (tail arguments ignored).
// Launched as a programmatic dependent of the previous kernel on the stream: its set-up overlaps that kernel's tail,
// and it waits for that kernel to complete before it touches anything.
// row_range (f32 output only, may be null): 2*M words, zeroed by the caller, that receive every output row's range as
// order-preserving keys -- see launch_quantize_rows_with_keys.  a_pieces > 1: A is stored as that many equal column
// blocks, block r a row-major [M, K / a_pieces] matrix at A + r * M * (K / a_pieces) (the layout an all-gather of
// column-sharded activations leaves); K / a_pieces must then be a multiple of 128.
int launch_gemm_i8_umma(b200q_ctx* ctx, const int8_t* A, const int8_t* W_nk, int64_t M, int64_t N, int64_t K,
                        const float* a_scales, const float* w_scales, const float* bias, int act, float* out_f32,
                        int32_t* out_i32, int8_t* out_q, double q_scale, uint32_t* row_range = nullptr, int a_pieces = 1);

// One thread waits with the tensor-core kernel's bounded wait on a barrier nothing signals (no asynchronous work in
// flight) and sets STATUS_SELFTEST_WAIT_TIMEOUT when the wait gives up.
int launch_selftest_bounded_wait(b200q_ctx* ctx, unsigned long long limit_ns);

// f32 pieces of a transformer block (block_kernels.cu).
int launch_embedding(b200q_ctx* ctx, const float* table, const int32_t* tokens, const float* pos_table, int64_t M, int64_t D,
                     int64_t V, int64_t S, float* out);
int launch_add_f32(b200q_ctx* ctx, const float* a, const float* b, int64_t n, float* out);
// y = LayerNorm(x [+ residual]); any of sum_out (x + residual), y_out (f32 result), q_out + scales_out (per-token codes) may be null.
int launch_layernorm_quantize(b200q_ctx* ctx, const float* x, const float* residual, const float* gamma, const float* beta,
                              float eps, int64_t M, int64_t D, float* sum_out, float* y_out, int8_t* q_out, float* scales_out);
int launch_sdpa_f32(b200q_ctx* ctx, const float* q, const float* k, const float* v, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                    int64_t B, int64_t H, int64_t S, int64_t Dh, float scale, int causal, float* out, int64_t ld_o);

// conv_group.cu: per-group (INT4-style) codes of a constant and the int8 convolution.
int launch_quantize_per_group(b200q_ctx* ctx, const float* x, int64_t n, int64_t group_size, int num_bits, int8_t* q,
                              double* scales64, float* scales32);
int launch_dequantize_per_group(b200q_ctx* ctx, const int8_t* q, int64_t n, int64_t group_size, const double* scales64, double* y64,
                                float* y32);
// layout 0: input / output NCHW, kernel OIHW; 1: input / output NHWC, kernel OHWI.  Uses the context's workspaces.
int launch_quantized_conv2d(b200q_ctx* ctx, const int8_t* in, const int8_t* ker, int64_t N, int64_t C, int64_t H, int64_t W, int64_t O,
                            int64_t KH, int64_t KW, int sh, int sw, int pt, int pb, int pl, int pr, int dh, int dw, int groups,
                            int zp_in, int zp_ker, int layout, int32_t* out);

// host_stage.cu: threads that copy between pageable host arrays and the page-locked staging ring.
struct HostStager;
HostStager* host_stager_create(int threads);
void host_stager_destroy(HostStager* s);
void host_stager_copy2(HostStager* s, void* d0, const void* s0, size_t n0, void* d1, const void* s1, size_t n1);

// api.cu: linear + per-token requantization of its result (see the definition).
int linear_requant_token_core(b200q_ctx* ctx, const int8_t* A, const float* a_scales, int a_pieces, const int8_t* W,
                              const float* w_scales, const float* bias, int act, int64_t M, int64_t N, int64_t K, float* y,
                              int8_t* out_q, int64_t ld_q, float* out_scales);

// Looks up (and caches) the device address of the fixed scratch array of b200q_linear_f32_noalloc for `device`, which
// must be current; called once per context at creation, so the array's module is loaded before any call needs it.
int noalloc_prepare(int device);

// attention_umma.cu: the same attention on the tensor cores (tcgen05.mma.kind::tf32, every product three ways).
bool sdpa_umma_supported(const float* q, const float* k, const float* v, const float* out, int64_t ld_q, int64_t ld_k, int64_t ld_v,
                         int64_t ld_o, int64_t B, int64_t H, int64_t S, int64_t Dh);
int launch_sdpa_umma(b200q_ctx* ctx, const float* q, const float* k, const float* v, int64_t ld_q, int64_t ld_k, int64_t ld_v, int64_t B,
                     int64_t H, int64_t S, float scale, int causal, float* out, int64_t ld_o);

}  // namespace b200q
