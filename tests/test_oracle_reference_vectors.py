"""Pins the CPU oracle against the known answers held by the reference's own tests.

Each test restates one reference test (cited by file:line inside the reference
project).  The reference stores no golden arrays for this path: its tests use
closed-form inputs (sines, small literals) and assert formulas, tolerances and
error ratios.  The same inputs and the same assertions are applied to the oracle.
"""
import math

import numpy as np
import pytest

SYM, ASYM, PERCH = 0, 1, 2
I8, UI8 = 0, 1


# tests/compiler/passes/quantization/params.test.js:6-23
def test_from_range_symmetric(orc):
    s, z = orc.from_range(-3, 3, SYM)
    assert s == pytest.approx(3 / 127, abs=1e-10) and z == 0
    s, _ = orc.from_range(-1, 5, SYM)
    assert s == pytest.approx(5 / 127, abs=1e-10)
    assert orc.clamp_range(SYM, I8, 8) == (-127, 127)


# params.test.js:26-41
def test_from_range_asymmetric(orc):
    s, z = orc.from_range(0, 6, ASYM)
    assert s == pytest.approx(6 / 255, abs=1e-10)
    assert -128 <= z <= 127
    assert orc.clamp_range(ASYM, UI8, 8) == (0, 255)
    assert orc.clamp_range(PERCH, I8, 8) == (-128, 127)


# params.test.js:44-73
def test_quantize_roundtrip_and_saturation(orc):
    s, z = orc.from_range(-6, 6, SYM)
    cmin, cmax = orc.clamp_range(SYM)
    q = orc.qp_quantize(3.5, s, z, cmin, cmax)
    assert abs(orc.qp_dequantize(q, s, z) - 3.5) < s
    s1, z1 = orc.from_range(-1, 1, SYM)
    assert orc.qp_quantize(1000, s1, z1, cmin, cmax) == cmax
    assert orc.qp_quantize(-1000, s1, z1, cmin, cmax) == cmin
    assert orc.qp_quantize(0, s1, z1, cmin, cmax) == 0
    s10, z10 = orc.from_range(-10, 10, SYM)
    for v in [0, 1.5, -3.7, 9.9, -10]:
        q = orc.qp_quantize(v, s10, z10, cmin, cmax)
        assert abs(orc.qp_dequantize(q, s10, z10) - v) < s10


# params.test.js:76-88
def test_from_constant_array(orc):
    s, _ = orc.from_constant_array([1.0, -2.0, 3.0, -0.5], SYM)
    assert s == pytest.approx(3 / 127, abs=1e-10)
    s, _ = orc.from_constant_array([5.0, 5.0, 5.0], SYM)
    assert s == pytest.approx(5.5 / 127, abs=1e-10)


# params.test.js:90-119
def test_default_activation(orc):
    s, z = orc.from_range(-6, 6, SYM)
    assert s == pytest.approx(6 / 127, abs=1e-10) and z == 0


# tests/compiler/passes/quantization/pass.test.js:100-114,236-251
def test_activation_scale_other_widths(orc):
    assert orc.from_range(-6, 6, SYM, I8, 16)[0] == pytest.approx(6 / 32767, rel=1e-12)
    assert orc.from_range(-6, 6, SYM, I8, 32)[0] == pytest.approx(6 / (2 ** 31 - 1), rel=1e-12)


# params.test.js:148-184
def test_per_channel_k4_n3(orc):
    K, N = 4, 3
    W = np.array([math.sin(k * 1.7 + n) * (n + 1) * 3 for k in range(K) for n in range(N)])
    sc = orc.per_channel_scales(W, (K, N), 1)
    for n in range(N):
        assert sc[n] == pytest.approx(np.abs(W.reshape(K, N)[:, n]).max() / 127, abs=1e-10)
    q = orc.quantize_per_channel(W, (K, N), 1, sc)
    d = orc.dequantize_per_channel(q, (K, N), 1, sc)
    err = np.abs(d - W.reshape(K, N))
    assert (err <= sc[None, :] / 2 + 1e-9).all()
    sc0 = orc.per_channel_scales(W, (K, N), 0)
    for k in range(K):
        assert sc0[k] == pytest.approx(np.abs(W.reshape(K, N)[k]).max() / 127, abs=1e-10)


# pass.test.js:461-491: compiled dequantize(quantize(x)) == qp.dequantize(qp.quantize(x)) within 1e-4, not identity
def test_fake_quant_is_lossy_and_matches_params_math(orc):
    s, z = orc.from_range(-6, 6, SYM)
    cmin, cmax = orc.clamp_range(SYM)
    data = np.array([3.5, -2.1, 5.9, 1.234, -5.9, 0.001], np.float32)
    out = orc.dequantize_static(orc.quantize_static(data, s, z), s, z)
    applied = False
    for i, v in enumerate([3.5, -2.1, 5.9, 1.234, -5.9, 0.001]):
        ref = orc.qp_dequantize(orc.qp_quantize(v, s, z, cmin, cmax), s, z)
        assert abs(out[i] - ref) < 1e-4
        assert abs(out[i] - v) <= s + 1e-6
        applied |= abs(out[i] - v) > 1e-6
    assert applied


def _int8_matmul(orc, A, W, K, N, a_scale, per_channel):
    """The graph pass.test.js:505-525 builds by hand, evaluated as the CPU target would."""
    if per_channel:
        wsc = orc.per_channel_scales(W, (K, N), 1)
        wq = orc.quantize_per_channel(W, (K, N), 1, wsc)
        sv = np.array([a_scale * wsc[n] for n in range(N)])
    else:
        ws, _ = orc.from_constant_array(W, SYM)
        cmin, cmax = orc.clamp_range(SYM)
        wq = np.array([orc.qp_quantize(v, ws, 0, cmin, cmax) for v in W], np.int8).reshape(K, N)
        sv = np.full(N, a_scale * ws)
    aq = orc.quantize_static(A, a_scale, 0)
    acc = orc.qdot_i32(aq, wq, "KN")
    return orc.epilogue_sv(acc, sv.astype(np.float32))


# pass.test.js:493-549
def test_per_channel_beats_per_tensor_m4_k8_n6(orc):
    M, K, N = 4, 8, 6
    A = np.array([math.sin(i * 0.7) for i in range(M * K)], np.float32).reshape(M, K)
    W = np.array([math.sin(k * 1.3 + n) * (n + 1) * 2 for k in range(K) for n in range(N)], np.float32)
    ref = A.astype(np.float64) @ W.astype(np.float64).reshape(K, N)
    a_scale = float(np.abs(A).max()) / 127 or 1e-10
    pt = np.abs(_int8_matmul(orc, A, W.astype(np.float64), K, N, a_scale, False) - ref).mean()
    pc = np.abs(_int8_matmul(orc, A, W.astype(np.float64), K, N, a_scale, True) - ref).mean()
    assert pc < pt and pt / pc > 1.5


# tests/e2e/cuda/training-quant.cuda.test.js:70-125: the CPU side of the CPU-vs-CUDA checks must be sane
@pytest.mark.parametrize("M,K,N,step,a_scale", [(4, 8, 6, 0.7, 0.05), (64, 128, 32, 0.3, 0.02)])
def test_training_quant_matmul_inputs(orc, M, K, N, step, a_scale):
    A = np.array([math.sin(i * step) for i in range(M * K)], np.float32).reshape(M, K)
    W = np.array([math.sin(i * 1.1) * 3 for i in range(K * N)], np.float32)
    out = _int8_matmul(orc, A, W.astype(np.float64), K, N, a_scale, False)
    ref = A.astype(np.float64) @ W.astype(np.float64).reshape(K, N)
    # int8 x int8 with these scales keeps a few percent of the float result's range
    assert np.abs(out - ref).max() < 0.05 * np.abs(ref).max() + 3 * a_scale * K
    assert np.isfinite(out).all()


def test_training_quant_fake_quant_n16(orc):
    s, z = orc.from_range(-6, 6, SYM)
    x = np.array([math.sin(i) * 3 for i in range(16)], np.float32)
    y = orc.dequantize_static(orc.quantize_static(x, s, z), s, z)
    assert np.abs(y - x).max() <= s / 2 + 1e-6


# ---------------------------------------------------------------- source-only rules
def test_js_round_ties_toward_plus_infinity(orc):
    for x, r in [(2.5, 3), (-2.5, -2), (0.5, 1), (-0.5, 0), (1.4999999999999998, 1), (-1.5, -1),
                 (0.49999999999999994, 0), (126.5, 127), (-126.5, -126)]:
        assert orc.js_round(x) == r
    assert math.isnan(orc.js_round(float("nan")))
    assert orc.js_round(float("inf")) == float("inf")


def test_static_quantize_special_values(orc):
    x = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1e30, -1e30], np.float32)
    q = orc.quantize_static(x, 6 / 127, 0)
    assert q.tolist() == [0, 127, -128, 0, 0, 127, -128]


def test_per_token_special_rows(orc):
    x = np.zeros((5, 8), np.float32)
    x[1] = 3.0                       # all-equal row: range widened by +-0.5
    x[2, 3] = np.nan                 # NaN is ignored by the range and its code stores as 0
    x[2, 0] = 2.0
    x[3, 1] = np.inf                 # non-finite max -> 1
    x[3, 2] = -4.0
    x[4] = np.nan                    # nothing finite: range [-1, 1]
    q, s64, s32 = orc.quantize_per_token(x, -128, 127)
    assert s64[0] == 0.5 / 127 and (q[0] == 0).all()
    assert s64[1] == 3.5 / 127 and (q[1] == orc.js_round(3.0 / (3.5 / 127))).all()
    assert s64[2] == 2.0 / 127 and q[2, 3] == 0 and q[2, 0] == 127
    assert s64[3] == 4.0 / 127 and q[3, 1] == 127 and q[3, 2] == -127
    assert s64[4] == 1.0 / 127 and (q[4] == 0).all()
    assert (s32 == s64.astype(np.float32)).all()


def test_mulberry32_first_values(orc):
    # values from evaluating src/util/random.ts:5-14 by hand for seed 0 and 1
    def mb(seed, n):
        a = seed & 0xFFFFFFFF
        out = []
        for _ in range(n):
            a = (a + 0x6D2B79F5) & 0xFFFFFFFF
            t = ((a ^ (a >> 15)) * (1 | a)) & 0xFFFFFFFF
            t = ((t + (((t ^ (t >> 7)) * (61 | t)) & 0xFFFFFFFF)) & 0xFFFFFFFF) ^ t
            out.append(((t ^ (t >> 14)) & 0xFFFFFFFF) / 4294967296)
        return out
    for seed in (0, 1, 12345, 0x9E3779B9):
        assert orc.rng_uniform(seed, 8).tolist() == mb(seed, 8)


def test_gelu_sigmoid_uses_1702(orc):
    # tests/compiler/passes/decompose/activation.test.js:153-163 pins the 1.702 coefficient
    y = np.linspace(-6, 6, 97).astype(np.float32)
    g = orc.activation(y, "gelu_sigmoid")
    ref = y.astype(np.float64) / (1 + np.exp(-1.702 * y.astype(np.float64)))
    assert np.abs(g - ref).max() < 1e-6
    s = orc.activation(y, "silu")
    assert np.abs(s - y.astype(np.float64) / (1 + np.exp(-y.astype(np.float64)))).max() < 1e-6
    assert (orc.activation(y, "relu") == np.maximum(y, 0)).all()
    t = orc.activation(y, "gelu_tanh")
    yy = y.astype(np.float64)
    assert np.abs(t - 0.5 * yy * (1 + np.tanh(0.7978845608028654 * (yy + 0.044715 * yy ** 3)))).max() < 2e-6


def test_minmax_calibration(orc):
    # src/compiler/analysis/calibration.ts:24-34,246-268: running min/max -> fromRange
    b1 = np.array([0.5, -2.0, np.nan], np.float32)
    b2 = np.array([3.0, 1.0], np.float32)
    mn, mx = orc.minmax_observe([b1, b2])
    assert (mn, mx) == (-2.0, 3.0)
    assert orc.from_range(mn, mx, SYM)[0] == 3.0 / 127


# params.test.js:204-234 -- INT4 group-wise quantization (both restatements)
def test_per_group_int4_known_answers(orc):
    from oracle import jsport as js
    N, G = 64, 16
    data = [math.sin(i * 0.9) * (1 + (i % G) * 0.1) for i in range(N)]
    qp = js.QuantizationParams.from_constant_array_per_group(data, G, "i8", 4)
    scales = orc.per_group_scales(np.array(data), G, 4)
    assert qp.scheme == js.PER_GROUP and qp.num_bits == 4 and len(qp.scale) == math.ceil(N / G) == len(scales)
    assert list(scales) == qp.scale
    q_js = qp.quantize_array_per_group(data)
    q = orc.quantize_per_group(np.array(data), G, scales, 4)
    assert list(q) == q_js and all(float(v).is_integer() and -7 <= v <= 7 for v in q_js)
    deq = orc.dequantize_per_group(q, G, scales)
    assert list(deq) == qp.dequantize_array_per_group(q_js)
    assert max(abs(d - x) for d, x in zip(deq, data)) <= max(scales) / 2 + 1e-9
    # beats per-tensor INT4 (params.test.js:225-233)
    pt = js.QuantizationParams.from_constant_array(data, js.PER_TENSOR_SYMMETRIC, "i8", 4)
    pt_err = max(abs(d - x) for d, x in zip(pt.dequantize_array(pt.quantize_array(data)), data))
    assert max(abs(d - x) for d, x in zip(deq, data)) < pt_err
