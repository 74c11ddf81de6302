"""Regenerates the golden fixtures of this directory:  python tests/golden/make_golden.py

Inputs are the closed-form ones the reference's own tests use (the reference stores no arrays for this path;
tests/compiler/passes/quantization/pass.test.js:461-549, tests/e2e/cuda/training-quant.cuda.test.js:70-125,
tests/compiler/passes/quantization/params.test.js:148-184 inside the reference project).  Outputs are what the CPU
oracle computes for them; the oracle itself is pinned to the formulas and thresholds those tests assert
(tests/test_oracle_reference_vectors.py).  The fixtures freeze that state: a later change of the oracle or of the
CUDA kernels that alters a single bit shows up against them.
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle as orc  # noqa: E402

ACTS = ["none", "relu", "gelu_sigmoid", "silu", "gelu_tanh"]


def int8_matmul_case(M, K, N, a_step, w_fn, a_scale, per_channel):
    A = np.array([math.sin(i * a_step) for i in range(M * K)], np.float32).reshape(M, K)
    W = np.array([w_fn(k, n) for k in range(K) for n in range(N)], np.float32).reshape(K, N)
    if a_scale is None:
        a_scale = float(np.abs(A).max()) / 127 or 1e-10
    if per_channel:
        wsc = orc.per_channel_scales(W.astype(np.float64), (K, N), 1)
        wq = orc.quantize_per_channel(W.astype(np.float64), (K, N), 1, wsc)
        sv = np.array([a_scale * s for s in wsc])
    else:
        ws, _ = orc.from_constant_array(W.astype(np.float64).reshape(-1))
        wq = np.array([orc.qp_quantize(float(v), ws, 0, -127, 127) for v in W.reshape(-1)], np.int8).reshape(K, N)
        sv = np.full(N, a_scale * ws)
    aq = orc.quantize_static(A, a_scale, 0)
    acc = orc.qdot_i32(aq, wq, "KN")
    out = orc.epilogue_sv(acc, sv.astype(np.float32))
    return dict(A=A, W=W, a_scale=np.float64(a_scale), wq=wq, sv=sv.astype(np.float32), aq=aq, acc=acc, out=out)


def main():
    # pass.test.js:493-549 (hand-built per-channel int8 matmul, M4 K8 N6)
    np.savez(os.path.join(HERE, "matmul_m4k8n6.npz"),
             **int8_matmul_case(4, 8, 6, 0.7, lambda k, n: math.sin(k * 1.3 + n) * (n + 1) * 2, None, True))
    # training-quant.cuda.test.js:86-124 (per-tensor weights, aScale given)
    np.savez(os.path.join(HERE, "matmul_m64k128n32.npz"),
             **int8_matmul_case(64, 128, 32, 0.3, lambda k, n: math.sin((k * 32 + n) * 1.1) * 3, 0.02, False))
    # pass.test.js:461-491 + training-quant fake-quant n=16: static quantize / dequantize at scale 6/127
    s, _ = orc.from_range(-6, 6)
    x = np.array([3.5, -2.1, 5.9, 1.234, -5.9, 0.001] + [math.sin(i) * 3 for i in range(16)] +
                 [(k + 0.5) * s for k in range(-6, 6)] + [float("nan"), float("inf"), float("-inf"), 0.0, -0.0, 1e30], np.float32)
    q = orc.quantize_static(x, s, 0)
    np.savez(os.path.join(HERE, "static_quant.npz"), x=x, scale=np.float64(s), q=q, y=orc.dequantize_static(q, s, 0))
    # per-token quantize of a [12, 40] tensor of sines with one constant row, one zero row and one row with a NaN
    xt = np.array([math.sin(0.37 * i) * (1 + (i % 7)) for i in range(12 * 40)], np.float32).reshape(12, 40)
    xt[3] = 2.5
    xt[5] = 0.0
    xt[7, 11] = np.nan
    qt, s64, s32 = orc.quantize_per_token(xt)
    np.savez(os.path.join(HERE, "per_token.npz"), x=xt, q=qt, scales64=s64, scales32=s32, y=orc.dequantize_per_token_f32(qt, s32))
    # one small linear with every tail (K multiple of 16 so that the tensor-core kernel takes it)
    M, K, N = 8, 64, 16
    xl = np.array([math.sin(0.11 * i) * 2 for i in range(M * K)], np.float32).reshape(M, K)
    wl = np.array([round(math.sin(0.23 * i) * 127) for i in range(N * K)], np.int8).reshape(N, K)
    ws = np.array([1e-3 * (1 + n) for n in range(N)], np.float32)
    bias = np.array([math.cos(n) * 0.1 for n in range(N)], np.float32)
    ql, _, sl = orc.quantize_per_token(xl)
    acc = orc.qdot_i32(ql, wl)
    outs = {f"out_{a}": orc.epilogue(acc, sl, ws, bias, a) for a in ACTS}
    np.savez(os.path.join(HERE, "linear_tails.npz"), x=xl, w=wl, w_scales=ws, bias=bias, q=ql, a_scales=sl, acc=acc, **outs)
    # f32 pieces of a transformer block on closed-form inputs: LayerNorm (with a residual) and causal attention,
    # 2 sequences x 24 positions, 2 heads of 64 -- outputs of the oracle's index-order binary32 restatement
    Mb, Db = 48, 128
    xb = np.array([math.sin(0.13 * i) * 2 + math.cos(0.07 * i) for i in range(Mb * Db)], np.float32).reshape(Mb, Db)
    rb = np.array([math.sin(0.31 * i) for i in range(Mb * Db)], np.float32).reshape(Mb, Db)
    gamma = np.array([1 + 0.5 * math.sin(d) for d in range(Db)], np.float32)
    beta = np.array([0.1 * math.cos(d) for d in range(Db)], np.float32)
    yb, sb = orc.layer_norm(xb, gamma, beta, 1e-5, add=rb, want_sum=True)
    qb = np.array([math.sin(0.17 * i) * 1.5 for i in range(Mb * Db)], np.float32).reshape(Mb, Db)
    kb = np.array([math.cos(0.19 * i) * 1.5 for i in range(Mb * Db)], np.float32).reshape(Mb, Db)
    vb = np.array([math.sin(0.23 * i + 1) for i in range(Mb * Db)], np.float32).reshape(Mb, Db)
    ab = orc.sdpa(qb, kb, vb, 2, 2, 24, 64, 0.125, True)
    np.savez(os.path.join(HERE, "block_ops.npz"), x=xb, residual=rb, gamma=gamma, beta=beta, ln_sum=sb, ln_out=yb,
             q=qb, k=kb, v=vb, attn=ab)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
