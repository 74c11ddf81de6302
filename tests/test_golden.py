"""Committed golden fixtures (tests/golden/*.npz, made by tests/golden/make_golden.py from the reference tests'
closed-form inputs with the pure-Python restatement oracle/jsport.py): the C++ oracle must reproduce them bit for bit
(CPU) - two independent restatements agreeing - and so must the CUDA path (GPU)."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
ACTS = ["none", "relu", "gelu_sigmoid", "silu", "gelu_tanh"]


def load(name):
    return dict(np.load(os.path.join(GOLD, name)))


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and a.dtype == b.dtype and (a.view(np.uint8) == b.view(np.uint8)).all()


def test_fixture_generator_uses_the_python_port_only():
    src = open(os.path.join(GOLD, "make_golden.py")).read()
    assert "from oracle import jsport" in src
    assert "import oracle as" not in src and "orc." not in src and "liboracle" not in src


# ------------------------------------------------------------------ CPU: the oracle against the fixtures
def test_oracle_reproduces_per_group_and_conv_fixtures(orc):
    g = load("per_group.npz")
    for tag in "abc":
        G, bits = (int(v) for v in g[f"meta_{tag}"])
        s = orc.per_group_scales(g[f"x_{tag}"], G, bits)
        assert same_bits(s, g[f"scales_{tag}"])
        q = orc.quantize_per_group(g[f"x_{tag}"], G, s, bits)
        assert same_bits(q, g[f"q_{tag}"])
        assert same_bits(orc.dequantize_per_group(q, G, s), g[f"deq_{tag}"])
    g = load("quantized_conv.npz")
    for tag in "ab":
        sh, sw, pt, pb, pl, pr, dh, dw, groups, zi, zk = (int(v) for v in g[f"geom_{tag}"])
        out = orc.quantized_conv2d(g[f"x_{tag}"], g[f"k_{tag}"], (sh, sw), ((pt, pb), (pl, pr)), (dh, dw), groups, zi, zk, "NCHW")
        assert same_bits(out, g[f"out_{tag}"])


def test_oracle_reproduces_matmul_fixtures(orc):
    for name in ("matmul_m4k8n6.npz", "matmul_m64k128n32.npz"):
        g = load(name)
        aq = orc.quantize_static(g["A"], float(g["a_scale"]), 0)
        assert same_bits(aq, g["aq"])
        acc = orc.qdot_i32(aq, g["wq"], "KN")
        assert same_bits(acc, g["acc"])
        assert same_bits(orc.epilogue_sv(acc, g["sv"]), g["out"])
        ref = g["A"].astype(np.float64) @ g["W"].astype(np.float64)
        K = g["A"].shape[1]
        assert np.abs(g["out"] - ref).max() < 0.05 * np.abs(ref).max() + 3 * float(g["a_scale"]) * K   # a sane int8 approximation


def test_oracle_reproduces_quantize_fixtures(orc):
    g = load("static_quant.npz")
    assert same_bits(orc.quantize_static(g["x"], float(g["scale"]), 0), g["q"])
    assert same_bits(orc.dequantize_static(g["q"], float(g["scale"]), 0), g["y"])
    g = load("per_token.npz")
    q, s64, s32 = orc.quantize_per_token(g["x"])
    assert same_bits(q, g["q"]) and same_bits(s64, g["scales64"]) and same_bits(s32, g["scales32"])
    assert same_bits(orc.dequantize_per_token_f32(q, s32), g["y"])
    assert g["scales64"][3] == 3.0 / 127 and g["scales64"][5] == 0.5 / 127 and g["q"][7, 11] == 0


def test_oracle_reproduces_linear_fixture(orc):
    g = load("linear_tails.npz")
    q, _, s = orc.quantize_per_token(g["x"])
    assert same_bits(q, g["q"]) and same_bits(s, g["a_scales"])
    acc = orc.qdot_i32(q, g["w"])
    assert same_bits(acc, g["acc"])
    for a in ACTS:
        assert same_bits(orc.epilogue(acc, s, g["w_scales"], g["bias"], a), g[f"out_{a}"])


def test_oracle_reproduces_block_fixture(orc):
    g = load("block_ops.npz")
    y, s = orc.layer_norm(g["x"], g["gamma"], g["beta"], 1e-5, add=g["residual"], want_sum=True)
    assert same_bits(y, g["ln_out"]) and same_bits(s, g["ln_sum"])
    assert same_bits(orc.sdpa(g["q"], g["k"], g["v"], 2, 2, 24, 64, 0.125, True), g["attn"])
    assert same_bits(g["attn"][0], g["v"][0]) and same_bits(g["attn"][24], g["v"][24])   # a first position attends to itself only


# ------------------------------------------------------------------ GPU: the CUDA path against the fixtures
@pytest.fixture(scope="module")
def ctx():
    import mlfw_b200
    c = mlfw_b200.Context(0)
    yield c
    c.check_status()
    c.close()


@pytest.mark.gpu
def test_cuda_matches_matmul_fixtures(ctx):
    for name in ("matmul_m4k8n6.npz", "matmul_m64k128n32.npz"):
        g = load(name)
        M, K = g["A"].shape
        N = g["W"].shape[1]
        dA = ctx.to_device(g["A"])
        dq = ctx.empty((M, K), np.int8)
        ctx.quantize_static(dA, M * K, float(g["a_scale"]), 0, 0, dq)
        dw_kn, dw_nk = ctx.to_device(g["wq"]), ctx.empty((N, K), np.int8)
        ctx.transpose_i8(dw_kn, K, N, dw_nk)
        dacc, dout, dsv = ctx.empty((M, N), np.int32), ctx.empty((M, N), np.float32), ctx.to_device(g["sv"])
        ctx.int8_gemm_i32(dq, dw_nk, M, N, K, dacc)
        ctx.int8_linear(dq, None, dw_nk, dsv, None, "none", M, N, K, dout)
        ctx.sync()
        assert same_bits(dq.download(), g["aq"]) and same_bits(dacc.download(), g["acc"]) and same_bits(dout.download(), g["out"])


@pytest.mark.gpu
def test_cuda_matches_quantize_fixtures(ctx):
    g = load("static_quant.npz")
    n = g["x"].size
    dx, dq, dy = ctx.to_device(g["x"]), ctx.empty((n,), np.int8), ctx.empty((n,), np.float32)
    ctx.quantize_static(dx, n, float(g["scale"]), 0, 0, dq)
    ctx.dequantize_static(dq, 0, n, float(g["scale"]), 0, dy)
    ctx.sync()
    assert same_bits(dq.download(), g["q"]) and same_bits(dy.download(), g["y"])
    g = load("per_token.npz")
    M, K = g["x"].shape
    dx, dq, ds, dy = ctx.to_device(g["x"]), ctx.empty((M, K), np.int8), ctx.empty((M,), np.float32), ctx.empty((M, K), np.float32)
    ctx.quantize_per_token(dx, M, K, dq, ds)
    ctx.dequantize_per_token(dq, ds, M, K, dy)
    ctx.sync()
    assert same_bits(dq.download(), g["q"]) and same_bits(ds.download(), g["scales32"]) and same_bits(dy.download(), g["y"])


@pytest.mark.gpu
@pytest.mark.parametrize("variant", [1, 2, 3])
def test_cuda_matches_linear_fixture(ctx, variant):
    g = load("linear_tails.npz")
    M, K = g["x"].shape
    N = g["w"].shape[0]
    dx, dw, dws, db = ctx.to_device(g["x"]), ctx.to_device(g["w"]), ctx.to_device(g["w_scales"]), ctx.to_device(g["bias"])
    ctx.set_gemm_variant(variant)
    try:
        for a in ACTS:
            dout = ctx.empty((M, N), np.float32)
            ctx.linear_f32(dx, dw, dws, db, a, M, N, K, dout)
            ctx.sync()
            out = dout.download()
            if a == "gelu_tanh":      # no reference form: tolerance only
                assert np.abs(out - g[f"out_{a}"]).max() <= 1e-5 * np.abs(g[f"out_{a}"]).max()
            else:
                assert same_bits(out, g[f"out_{a}"]), a
    finally:
        ctx.set_gemm_variant(0)


@pytest.mark.gpu
def test_cuda_matches_block_fixture(ctx):
    """Floating-point reductions: within 1e-5 of the output's largest magnitude; the residual sum bit for bit."""
    g = load("block_ops.npz")
    M, D = g["x"].shape
    dsum, dy = ctx.empty((M, D), np.float32), ctx.empty((M, D), np.float32)
    ctx.layernorm_quantize(ctx.to_device(g["x"]), ctx.to_device(g["residual"]), ctx.to_device(g["gamma"]), ctx.to_device(g["beta"]),
                           1e-5, M, D, dsum, dy, None, None)
    dattn = ctx.empty((M, D), np.float32)
    ctx.sdpa_f32(ctx.to_device(g["q"]), ctx.to_device(g["k"]), ctx.to_device(g["v"]), D, D, D, 2, 2, 24, 64, 0.125, True, dattn, D)
    ctx.sync()
    assert same_bits(dsum.download(), g["ln_sum"])
    assert np.abs(dy.download() - g["ln_out"]).max() <= 1e-5 * np.abs(g["ln_out"]).max()
    assert np.abs(dattn.download() - g["attn"]).max() <= 1e-5 * np.abs(g["attn"]).max()


@pytest.mark.gpu
def test_cuda_matches_per_group_and_conv_fixtures(ctx):
    g = load("per_group.npz")
    for tag in "abc":
        G, bits = (int(v) for v in g[f"meta_{tag}"])
        x = g[f"x_{tag}"]
        n, groups = x.size, (x.size + G - 1) // G
        dq, ds = ctx.empty((n,), np.int8), ctx.empty((groups,), np.float64)
        ctx.quantize_per_group(ctx.to_device(x), n, G, bits, dq, ds, None)
        dy = ctx.empty((n,), np.float64)
        ctx.dequantize_per_group(dq, n, G, ds, dy, None)
        ctx.sync()
        assert same_bits(ds.download(), g[f"scales_{tag}"]) and same_bits(dq.download(), g[f"q_{tag}"]) and same_bits(dy.download(), g[f"deq_{tag}"])
    g = load("quantized_conv.npz")
    for tag in "ab":
        sh, sw, pt, pb, pl, pr, dh, dw, groups, zi, zk = (int(v) for v in g[f"geom_{tag}"])
        x, k, ref = g[f"x_{tag}"], g[f"k_{tag}"], g[f"out_{tag}"]
        do = ctx.empty(ref.shape, np.int32)
        ctx.quantized_conv2d(ctx.to_device(x), ctx.to_device(k), x.shape, (k.shape[0], k.shape[2], k.shape[3]), do, (sh, sw), ((pt, pb), (pl, pr)),
                             (dh, dw), groups, zi, zk, "NCHW")
        ctx.sync()
        assert same_bits(do.download(), ref)
