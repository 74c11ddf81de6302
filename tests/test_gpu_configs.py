"""The five benchmark configurations at their full sizes on the GPU.

Where the CPU oracle cannot evaluate a whole tensor in seconds, rows are sampled: every output row of the path
depends only on its own input row and the replicated weights, so the oracle's result for a subset of rows is the
exact expectation for those rows.  The tensor-core kernel is additionally cross-checked against the CUDA-core
kernel on the whole int32 accumulator (both on the device)."""
import numpy as np
import pytest

from gpu_util import rel_err
from mlfw_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-5
seed = synth.tensor_seed


@pytest.fixture(scope="module")
def ctx():
    import mlfw_b200
    c = mlfw_b200.Context(0)
    yield c
    c.check_status()
    c.close()


def sample_rows(M, n=48, s=0):
    rng = np.random.default_rng(s)
    rows = np.unique(np.concatenate([[0, 1, 127, 128, 255, 256, M - 1], rng.integers(0, M, n)]))
    return rows[rows < M]


def test_c2_roundtrip_16384x4096(ctx, orc):
    """Config 2 in full: f32 [16384,4096] ~ N(0,1), 0.1 % outliers ~ N(0,20); every code and scale bit-exact."""
    M, K = 16384, 4096
    x = synth.with_outliers(synth.normal(seed(0, 20), (M, K)), seed(0, 21), seed(0, 22))
    dx, dq, ds, dy = ctx.to_device(x), ctx.empty((M, K), np.int8), ctx.empty((M,), np.float32), ctx.empty((M, K), np.float32)
    ctx.quantize_per_token(dx, M, K, dq, ds)
    ctx.dequantize_per_token(dq, ds, M, K, dy)
    ctx.sync()
    q, s, y = dq.download(), ds.download(), dy.download()
    rq, s64, rs = orc.quantize_per_token(x)
    assert (s.view(np.uint32) == rs.view(np.uint32)).all()
    assert (q == rq).all()
    assert (y.view(np.uint32) == orc.dequantize_per_token_f32(rq, rs).view(np.uint32)).all()
    assert rel_err(y, orc.dequantize_per_channel(rq, (M, K), 0, s64)) <= TOL          # the reference's binary64 dequantize
    # round trip within half a step (plus the two binary32 roundings of the dequantized value)
    assert (np.abs(y.astype(np.float64) - x) <= s64[:, None] / 2 + 2.0 ** -22 * np.abs(y) + 1e-9).all()
    assert np.abs(q).max() == 127 and (np.abs(q).max(axis=1) == 127).all()           # every row uses its full range


@pytest.mark.parametrize("act", ["gelu_tanh", "gelu_sigmoid"])
def test_c3_gemm_8192x4096x4096(ctx, orc, act):
    """Config 3 in full: activations N(0,1) quantized per token, int8 weights uniform in [-127,127], per-channel scales
    U(1e-3,1e-2), bias N(0,0.01), GELU epilogue (tanh as the benchmark definition words it, sigmoid as the reference implements it)."""
    M, K, N = 8192, 4096, 4096
    x = synth.normal(seed(0, 100), (M, K))
    W = synth.randint_i8(seed(0, 1), (N, K))
    ws = synth.uniform(seed(0, 2), (N,), 1e-3, 1e-2)
    bias = synth.normal(seed(0, 3), (N,), 0.0, 0.01)
    dx, dW, dws, db = ctx.to_device(x), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    dq, ds = ctx.empty((M, K), np.int8), ctx.empty((M,), np.float32)
    dout, dacc, dacc2 = ctx.empty((M, N), np.float32), ctx.empty((M, N), np.int32), ctx.empty((M, N), np.int32)
    ctx.quantize_per_token(dx, M, K, dq, ds)
    ctx.linear_f32(dx, dW, dws, db, act, M, N, K, dout)
    ctx.int8_gemm_i32(dq, dW, M, N, K, dacc)
    ctx.set_gemm_variant(1)
    ctx.int8_gemm_i32(dq, dW, M, N, K, dacc2)
    ctx.set_gemm_variant(0)
    ctx.sync()
    acc = dacc.download()
    assert (acc == dacc2.download()).all()                       # tensor cores == CUDA cores on all 33.5 M accumulators
    rows = sample_rows(M)
    out, q, s = dout.download()[rows], dq.download()[rows], ds.download()[rows]
    ref, rq, rs, racc = orc.linear(x[rows], W, ws, bias, act)
    assert (q == rq).all() and (s == rs).all() and (acc[rows] == racc).all()
    assert rel_err(out, ref) <= TOL
    if act == "gelu_sigmoid":
        assert (out.view(np.uint32) == ref.view(np.uint32)).all()


def test_c4_gpt_block_linears(ctx, orc):
    """Config 4's int8 linears at full size (d_model 768, d_ff 3072, 32 x 512 = 16384 tokens): QKV, attention output,
    FC1 with the reference's GELU, FC2.  Weights ~ N(0,0.02) quantized per output channel on the device."""
    M, D, F = 16384, 768, 3072
    x = synth.normal(seed(4, 0), (M, D))
    rows = sample_rows(M, 24)
    dx = ctx.to_device(x)
    specs = [("q", D, D, "none"), ("k", D, D, "none"), ("v", D, D, "none"), ("o", D, D, "none"), ("fc1", F, D, "gelu_sigmoid")]
    h_dev = None
    for i, (name, N, K, act) in enumerate(specs):
        w = synth.normal(seed(4, 10 + i), (N, K), 0.0, 0.02)          # [out, in], the layout of nn.Linear
        bias = synth.normal(seed(4, 30 + i), (N,), 0.0, 0.02)
        dw, dqw, dws, db = ctx.to_device(w), ctx.empty((N, K), np.int8), ctx.empty((N,), np.float32), ctx.to_device(bias)
        ctx.quantize_weights_per_channel(dw, N, K, 0, dqw, dws)
        dout = ctx.empty((M, N), np.float32)
        ctx.linear_f32(dx, dqw, dws, db, act, M, N, K, dout)
        ctx.sync()
        wsc = orc.per_channel_scales(w, (N, K), 0)
        wq = orc.quantize_per_channel(w, (N, K), 0, wsc, -128, 127)
        assert (dqw.download() == wq).all() and (dws.download() == wsc.astype(np.float32)).all()
        ref, _, _, _ = orc.linear(x[rows], wq, wsc.astype(np.float32), bias, act)
        out = dout.download()
        assert (out[rows].view(np.uint32) == ref.view(np.uint32)).all(), name
        # every output of the layer: the fused tensor-core path against the CUDA-core contraction + separate tail kernel
        dout2 = ctx.empty((M, N), np.float32)
        ctx.set_gemm_variant(1)
        ctx.linear_f32(dx, dqw, dws, db, act, M, N, K, dout2)
        ctx.set_gemm_variant(0)
        ctx.sync()
        assert (dout2.download().view(np.uint32) == out.view(np.uint32)).all(), name
        dout2.free()
        # the float model is approximated to about a percent
        yf = x[rows].astype(np.float64) @ w.T.astype(np.float64) + bias
        if act == "none":
            assert np.abs(out[rows] - yf).sum() / np.abs(yf).sum() < 0.02
        if name == "fc1":
            h_dev, h_host = dout, out
    # FC2 on FC1's output, K = 3072
    w2 = synth.normal(seed(4, 20), (D, F), 0.0, 0.02)
    b2 = synth.normal(seed(4, 40), (D,), 0.0, 0.02)
    dw2, dqw2, dws2, db2 = ctx.to_device(w2), ctx.empty((D, F), np.int8), ctx.empty((D,), np.float32), ctx.to_device(b2)
    ctx.quantize_weights_per_channel(dw2, D, F, 0, dqw2, dws2)
    dy = ctx.empty((M, D), np.float32)
    ctx.linear_f32(h_dev, dqw2, dws2, db2, "none", M, D, F, dy)
    ctx.sync()
    ref, _, _, _ = orc.linear(h_host[rows], dqw2.download(), dws2.download(), b2, "none")
    y_host = dy.download()
    assert (y_host[rows].view(np.uint32) == ref.view(np.uint32)).all()
    dy2 = ctx.empty((M, D), np.float32)
    ctx.set_gemm_variant(1)
    ctx.linear_f32(h_dev, dqw2, dws2, db2, "none", M, D, F, dy2)
    ctx.set_gemm_variant(0)
    ctx.sync()
    assert (dy2.download().view(np.uint32) == y_host.view(np.uint32)).all()


def test_c5_wide_projection_pair(ctx, orc):
    """Config 5's shapes: up-projection 8192 -> 28672 with SiLU and the per-token requantize of the next layer, then the
    down-projection 28672 -> 8192; M = 4096 rows, int8 weights uniform in [-127,127], scales U(1e-3,1e-2)/sqrt(K)."""
    M, K, N = 4096, 8192, 28672
    x = synth.normal(seed(5, 0), (M, K))
    W1 = synth.randint_i8(seed(5, 1), (N, K))
    W2 = synth.randint_i8(seed(5, 2), (K, N))
    ws1 = (synth.uniform(seed(5, 3), (N,), 1e-3, 1e-2) / np.sqrt(K)).astype(np.float32)
    ws2 = (synth.uniform(seed(5, 4), (K,), 1e-3, 1e-2) / np.sqrt(N)).astype(np.float32)
    dx, dW1, dW2, dws1, dws2 = ctx.to_device(x), ctx.to_device(W1), ctx.to_device(W2), ctx.to_device(ws1), ctx.to_device(ws2)
    dq, ds = ctx.empty((M, K), np.int8), ctx.empty((M,), np.float32)
    dh, dhs = ctx.empty((M, N), np.int8), ctx.empty((M,), np.float32)
    dy = ctx.empty((M, K), np.float32)
    ctx.quantize_per_token(dx, M, K, dq, ds)
    ctx.int8_linear_requant_token(dq, ds, dW1, dws1, None, "silu", M, N, K, dh, dhs)
    ctx.int8_linear(dh, dhs, dW2, dws2, None, "none", M, K, N, dy)
    ctx.sync()
    ctx.check_status()
    rows = sample_rows(M, 6)[:10]
    h_ref, q_ref, s_ref, _ = orc.linear(x[rows], W1, ws1, None, "silu")
    hq_ref, _, hs_ref = orc.quantize_per_token(h_ref)
    assert (dq.download()[rows] == q_ref).all()
    assert (dh.download()[rows] == hq_ref).all() and (dhs.download()[rows] == hs_ref).all()     # int8 codes through the chain
    y_ref = orc.epilogue(orc.qdot_i32(hq_ref, W2), hs_ref, ws2, None, "none")
    assert (dy.download()[rows].view(np.uint32) == y_ref.view(np.uint32)).all()
    # every accumulator of both layers: the tensor-core kernel against the CUDA-core (dp4a) kernel on the same codes
    for (a, w, n_out, k_in) in ((dq, dW1, N, K), (dh, dW2, K, N)):
        acc_t, acc_s = ctx.empty((M, n_out), np.int32), ctx.empty((M, n_out), np.int32)
        ctx.set_gemm_variant(0)
        ctx.int8_gemm_i32(a, w, M, n_out, k_in, acc_t)
        ctx.set_gemm_variant(1)
        ctx.int8_gemm_i32(a, w, M, n_out, k_in, acc_s)
        ctx.set_gemm_variant(0)
        ctx.sync()
        assert (acc_t.download() == acc_s.download()).all()
        acc_t.free(); acc_s.free()
    ctx.check_status()
