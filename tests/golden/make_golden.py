"""Regenerates the golden fixtures of this directory:  python tests/golden/make_golden.py

Inputs are the closed-form ones the reference's own tests use (the reference stores no arrays for this path;
tests/compiler/passes/quantization/pass.test.js:461-549, tests/e2e/cuda/training-quant.cuda.test.js:70-125,
tests/compiler/passes/quantization/params.test.js:148-184 inside the reference project).  Outputs are computed by
``oracle/jsport.py`` - the pure-Python, line-by-line restatement of the reference's TypeScript - and by nothing else:
the C++ oracle is not imported here.  ``tests/test_golden.py`` then holds the C++ oracle (CPU) and the CUDA path (GPU)
to these values bit for bit, so the fixtures are a check of both against an independent restatement, not a snapshot of
either.  numpy only packs the results.
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import jsport as js  # noqa: E402   (the Python port only; importing the package builds nothing)

ACTS = ["none", "relu", "gelu_sigmoid", "silu", "gelu_tanh"]


def f32(v):
    return js.fround(v)


def int8_matmul_case(M, K, N, a_step, w_fn, a_scale, per_channel):
    A = [[f32(math.sin((m * K + k) * a_step)) for k in range(K)] for m in range(M)]
    W = [[f32(w_fn(k, n)) for n in range(N)] for k in range(K)]                     # [K, N], as the reference's tests build it
    if a_scale is None:
        a_scale = js.js_or(max(abs(v) for r in A for v in r) / 127, 1e-10)
    flat_w = [v for r in W for v in r]
    if per_channel:
        wp = js.QuantizationParams.from_constant_array_per_channel(flat_w, [K, N], 1)
        codes = wp.quantize_array_per_channel(flat_w, [K, N])
        wq = [[js.to_int8(codes[k * N + n]) for n in range(N)] for k in range(K)]
        sv = [a_scale * s for s in wp.scale]                                          # binary64 products, stored as f32 below
    else:
        wp = js.QuantizationParams.from_constant_array(flat_w, js.PER_TENSOR_SYMMETRIC)
        wq = [[js.to_int8(wp.quantize(W[k][n])) for n in range(N)] for k in range(K)]
        sv = [a_scale * wp.scale] * N
    aq = [[js.compiled_quantize(v, a_scale, 0) for v in r] for r in A]
    w_nk = [[wq[k][n] for k in range(K)] for n in range(N)]
    acc = js.quantized_dot(aq, w_nk)
    sv32 = [f32(v) for v in sv]
    out = js.tail_sv(acc, sv32, None, "none")
    return dict(A=np.array(A, np.float32), W=np.array(W, np.float32), a_scale=np.float64(a_scale), wq=np.array(wq, np.int8),
                sv=np.array(sv32, np.float32), aq=np.array(aq, np.int8), acc=np.array(acc, np.int32), out=np.array(out, np.float32))


def main():
    # pass.test.js:493-549 (hand-built per-channel int8 matmul, M4 K8 N6)
    np.savez(os.path.join(HERE, "matmul_m4k8n6.npz"),
             **int8_matmul_case(4, 8, 6, 0.7, lambda k, n: math.sin(k * 1.3 + n) * (n + 1) * 2, None, True))
    # training-quant.cuda.test.js:86-124 (per-tensor weights, aScale given)
    np.savez(os.path.join(HERE, "matmul_m64k128n32.npz"),
             **int8_matmul_case(64, 128, 32, 0.3, lambda k, n: math.sin((k * 32 + n) * 1.1) * 3, 0.02, False))
    # pass.test.js:461-491 + training-quant fake-quant n=16: static quantize / dequantize at scale 6/127
    s = js.QuantizationParams.from_range(-6, 6, js.PER_TENSOR_SYMMETRIC).scale
    x = [f32(v) for v in [3.5, -2.1, 5.9, 1.234, -5.9, 0.001] + [math.sin(i) * 3 for i in range(16)] +
         [(k + 0.5) * s for k in range(-6, 6)] + [float("nan"), float("inf"), float("-inf"), 0.0, -0.0, 1e30]]
    q = [js.compiled_quantize(v, s, 0) for v in x]
    np.savez(os.path.join(HERE, "static_quant.npz"), x=np.array(x, np.float32), scale=np.float64(s), q=np.array(q, np.int8),
             y=np.array([js.compiled_dequantize(c, s, 0) for c in q], np.float32))
    # per-token quantize of a [12, 40] tensor of sines with one constant row, one zero row and one row with a NaN
    xt = [[f32(math.sin(0.37 * (m * 40 + k)) * (1 + ((m * 40 + k) % 7))) for k in range(40)] for m in range(12)]
    xt[3] = [2.5] * 40
    xt[5] = [0.0] * 40
    xt[7][11] = float("nan")
    qt, s64, s32 = js.quantize_per_token(xt)
    np.savez(os.path.join(HERE, "per_token.npz"), x=np.array(xt, np.float32), q=np.array(qt, np.int8), scales64=np.array(s64, np.float64),
             scales32=np.array(s32, np.float32), y=np.array(js.dequantize_per_token_f32(qt, s32), np.float32))
    # one small linear with every tail (K multiple of 16 so that the tensor-core kernel takes it)
    M, K, N = 8, 64, 16
    xl = [[f32(math.sin(0.11 * (m * K + k)) * 2) for k in range(K)] for m in range(M)]
    wl = [[js.to_int8(float(round(math.sin(0.23 * (n * K + k)) * 127))) for k in range(K)] for n in range(N)]
    ws = [f32(1e-3 * (1 + n)) for n in range(N)]
    bias = [f32(math.cos(n) * 0.1) for n in range(N)]
    ql, _, sl = js.quantize_per_token(xl)
    acc = js.quantized_dot(ql, wl)
    outs = {f"out_{a}": np.array(js.tail(acc, sl, ws, bias, a), np.float32) for a in ACTS}
    np.savez(os.path.join(HERE, "linear_tails.npz"), x=np.array(xl, np.float32), w=np.array(wl, np.int8), w_scales=np.array(ws, np.float32),
             bias=np.array(bias, np.float32), q=np.array(ql, np.int8), a_scales=np.array(sl, np.float32), acc=np.array(acc, np.int32), **outs)
    # f32 pieces of a transformer block on closed-form inputs: LayerNorm (with a residual) and causal attention,
    # 2 sequences x 24 positions, 2 heads of 64 -- index-order binary32 arithmetic
    Mb, Db = 48, 128
    grid = lambda fn: [[f32(fn(m * Db + d)) for d in range(Db)] for m in range(Mb)]
    xb = grid(lambda i: math.sin(0.13 * i) * 2 + math.cos(0.07 * i))
    rb = grid(lambda i: math.sin(0.31 * i))
    gamma = [f32(1 + 0.5 * math.sin(d)) for d in range(Db)]
    beta = [f32(0.1 * math.cos(d)) for d in range(Db)]
    yb, sb = js.layer_norm(xb, gamma, beta, 1e-5, add=rb)
    qb = grid(lambda i: math.sin(0.17 * i) * 1.5)
    kb = grid(lambda i: math.cos(0.19 * i) * 1.5)
    vb = grid(lambda i: math.sin(0.23 * i + 1))
    ab = js.sdpa(qb, kb, vb, 2, 2, 24, 64, 0.125, True)
    a32 = lambda v: np.array(v, np.float32)
    np.savez(os.path.join(HERE, "block_ops.npz"), x=a32(xb), residual=a32(rb), gamma=a32(gamma), beta=a32(beta), ln_sum=a32(sb), ln_out=a32(yb),
             q=a32(qb), k=a32(kb), v=a32(vb), attn=a32(ab))
    # per-group INT4 on the reference test's own data (tests/compiler/passes/quantization/params.test.js:204-207) and on a
    # longer closed-form array with a ragged last group, a zero group and 3-bit codes
    pg = {}
    for tag, n, G, bits in (("a", 64, 16, 4), ("b", 203, 32, 4), ("c", 96, 8, 3)):
        data = [f32(math.sin(i * 0.9) * (1 + (i % G) * 0.1)) for i in range(n)]
        if tag == "b":
            data[64:96] = [0.0] * 32
        qp = js.QuantizationParams.from_constant_array_per_group(data, G, "i8", bits)
        q = qp.quantize_array_per_group(data)
        pg.update({f"x_{tag}": np.array(data, np.float32), f"meta_{tag}": np.array([G, bits], np.int64),
                   f"scales_{tag}": np.array(qp.scale, np.float64), f"q_{tag}": np.array([js.to_int8(v) for v in q], np.int8),
                   f"deq_{tag}": np.array(qp.dequantize_array_per_group(q), np.float64)})
    np.savez(os.path.join(HERE, "per_group.npz"), **pg)
    # quantized_conv on closed-form int8 codes: strides, uneven padding, dilation, two groups, both zero-points; and a
    # plain 3x3 / padding 1 layer with 16 taps per group so that the tensor-core contraction is the one checked
    cv = {}
    for tag, (N, C, H, W, O, KH, KW, st, pad, dil, groups, zi, zk) in (
            ("a", (2, 4, 7, 6, 6, 3, 3, (2, 1), ((1, 0), (2, 1)), (1, 2), 2, 3, -2)),
            ("b", (1, 16, 6, 6, 8, 3, 3, (1, 1), ((1, 1), (1, 1)), (1, 1), 1, 0, 0))):
        code = lambda i, f: int(js.math_round(127 * math.sin(f * i + 0.5)))
        x = [[[[code(((n * C + c) * H + h) * W + w, 0.37) for w in range(W)] for h in range(H)] for c in range(C)] for n in range(N)]
        k = [[[[code(((o * (C // groups) + c) * KH + a) * KW + b, 0.11) for b in range(KW)] for a in range(KH)] for c in range(C // groups)]
             for o in range(O)]
        out = js.quantized_conv2d(x, k, st, pad, dil, groups, zi, zk)
        cv.update({f"x_{tag}": np.array(x, np.int8), f"k_{tag}": np.array(k, np.int8), f"out_{tag}": np.array(out, np.int32),
                   f"geom_{tag}": np.array([st[0], st[1], pad[0][0], pad[0][1], pad[1][0], pad[1][1], dil[0], dil[1], groups, zi, zk], np.int64)})
    np.savez(os.path.join(HERE, "quantized_conv.npz"), **cv)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
