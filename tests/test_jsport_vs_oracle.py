"""Two independent restatements of the reference's CPU arithmetic must agree bit for bit.

``oracle/oracle.cpp`` (C++) and ``oracle/jsport.py`` (pure Python, one line per line of the TypeScript) were written
separately from the same sources.  Wherever the reference's own tests hold no stored values - exact ties, NaN and
infinite inputs, the 1e-10 fallback, the places where Math.fround lands in the tail - agreement between the two is what
pins the C++ oracle the GPU tests use.  At least 10^6 random values per quantization mode, every constructed edge case
of the GPU tests, the tail with all activations, and the f32 block pieces."""
import math
import struct

import numpy as np
import pytest

from oracle import jsport as js


def f32_list(a):
    return [float(v) for v in np.asarray(a, np.float32).reshape(-1)]


def bits32(vals):
    return np.array(vals, np.float32).view(np.uint32)


def same_f32(got, ref):
    """Bit-equal binary32 values; a NaN equals any NaN (a JavaScript number has one NaN: sign and payload are not
    observable in the reference, and the two restatements are free to differ in them)."""
    g = np.array(got, np.float32).reshape(-1)
    r = np.asarray(ref, np.float32).reshape(-1)
    return bool(((g.view(np.uint32) == r.view(np.uint32)) | (np.isnan(g) & np.isnan(r))).all())


def neighbours(v, n=1):
    """v and its n binary32 neighbours on either side (through zero into the denormals of the other sign)."""
    f = np.float32(v)
    below, above = [], []
    a = b = f
    for _ in range(n):
        a = np.nextafter(a, np.float32(-np.inf))
        b = np.nextafter(b, np.float32(np.inf))
        below.append(float(a))
        above.append(float(b))
    return below[::-1] + [float(f)] + above


# --------------------------------------------------------------------------------------------------- number semantics
def test_number_semantics_known_answers():
    assert js.math_round(2.5) == 3 and js.math_round(-2.5) == -2 and js.math_round(-0.5) == 0 and js.math_round(0.49999999999999994) == 0
    assert js.math_round(-3.5000000000000004) == -4 and js.math_round(1e300) == 1e300 and math.isnan(js.math_round(js.NAN))
    assert js.fround(0.1) == struct.unpack("<f", struct.pack("<f", 0.1))[0] and js.fround(1e39) == js.INF and js.fround(-1e39) == -js.INF
    assert js.fround(3.4028235677973366e38) == js.INF                     # the midpoint above the largest binary32 rounds to even = infinity
    assert js.to_int32(2 ** 31) == -2 ** 31 and js.to_int32(-1.9) == -1 and js.to_int32(js.NAN) == 0 and js.to_int32(js.INF) == 0
    assert js.to_int8(127.0) == 127 and js.to_int8(128.0) == -128 and js.to_int8(-129.0) == 127 and js.to_int8(js.NAN) == 0
    assert math.isnan(js.math_max(1.0, js.NAN)) and math.isnan(js.math_min(js.NAN, 1.0))
    assert js.js_or(0.0, 7.0) == 7.0 and js.js_or(-0.0, 7.0) == 7.0 and js.js_or(js.NAN, 7.0) == 7.0 and js.js_or(2.0, 7.0) == 2.0


def test_js_round_agrees(orc):
    rng = np.random.default_rng(0)
    vals = list(rng.standard_normal(20000) * 100) + [k + 0.5 for k in range(-300, 300)] + [math.nextafter(k + 0.5, d) for k in range(-50, 50) for d in (-1e9, 1e9)]
    for v in vals:
        assert orc.js_round(float(v)) == js.math_round(float(v))


# --------------------------------------------------------------------------------------------------- mode P (per token)
def special_rows(K):
    rng = np.random.default_rng(5)
    rows = []
    base = rng.standard_normal(K).astype(np.float32)
    rows.append(np.full(K, 2.5, np.float32))                              # constant: range widened by +-0.5
    rows.append(np.zeros(K, np.float32))
    rows.append(np.full(K, -0.0, np.float32))
    r = base.copy(); r[3] = np.nan; rows.append(r)                        # NaN ignored by the range, stored as 0
    rows.append(np.full(K, np.nan, np.float32))                           # nothing seen: range -1 .. 1
    r = base.copy(); r[5] = np.inf; rows.append(r)                        # non-finite end replaced by 1
    r = base.copy(); r[5] = -np.inf; r[6] = np.inf; rows.append(r)
    r = base.copy(); r[0] = 3e38; rows.append(r)
    r = (base * 1e-42).astype(np.float32); rows.append(r)                 # denormals
    r = (base * 1e-30).astype(np.float32); rows.append(r)
    # constructed ties: (q + 0.5) * scale and its neighbours, for a row whose absmax fixes the scale
    absmax = np.float32(3.0)
    s = float(absmax) / 127
    tie = []
    for q in range(-127, 127):
        tie += neighbours(js.fround((q + 0.5) * s))
    tie = (tie + [0.0] * K)[:K - 1]
    rows.append(np.array(tie + [float(absmax)], np.float32))
    return np.stack(rows)


def test_per_token_quantize_agrees_on_a_million_values_and_every_edge_case(orc):
    rng = np.random.default_rng(1)
    K = 1024
    x = rng.standard_normal((980, K)).astype(np.float32)
    mask = rng.random(x.shape) < 0.001
    x[mask] = (rng.standard_normal(int(mask.sum())) * 20).astype(np.float32)
    x = np.concatenate([x, special_rows(K)])
    assert x.size >= 10 ** 6
    q, s64, s32 = orc.quantize_per_token(x)
    jq, js64, js32 = js.quantize_per_token([f32_list(r) for r in x])
    assert (np.array(js64, np.float64).view(np.uint64) == s64.view(np.uint64)).all()
    assert (bits32(js32) == s32.view(np.uint32)).all()
    assert (np.array(jq, np.int8) == q).all()
    # dequantize with the binary32 scales
    y = orc.dequantize_per_token_f32(q[:64], s32[:64])
    jy = js.dequantize_per_token_f32(jq[:64], js32[:64])
    assert (bits32(jy).reshape(y.shape) == y.view(np.uint32)).all()


def test_quantization_params_scalar_api_agrees(orc):
    rng = np.random.default_rng(2)
    for scheme, oscheme in ((js.PER_TENSOR_SYMMETRIC, 0), (js.PER_TENSOR_ASYMMETRIC, 1)):
        for dtype, odt in (("i8", 0), ("ui8", 1)):
            for mn, mx in [(-6.0, 6.0), (-1.0, 3.0), (0.0, 0.0), (2.0, 2.0), (-1e-12, 1e-12), (0.5, 7.25)]:
                p = js.QuantizationParams.from_range(mn, mx, scheme, dtype)
                s, zp = orc.from_range(mn, mx, oscheme, odt)
                assert p.scale == s and p.zero_point == zp
                c0, c1 = orc.clamp_range(oscheme, odt)
                assert p.clamp_range() == [c0, c1]
                for v in list(rng.standard_normal(200) * 4) + [0.0, mn, mx, 1e9, -1e9, float("nan"), (0.5 - zp) * s, (1.5 - zp) * s, (-0.5 - zp) * s]:
                    a, b = p.quantize(float(v)), orc.qp_quantize(float(v), s, zp, c0, c1)
                    assert (a == b) or (a != a and b != b)
                    if a == a:
                        assert p.dequantize(a) == orc.qp_dequantize(a, s, zp)
    data = list(rng.standard_normal(50))
    for d in (data, [4.0] * 7, [float("nan"), 1.0, -2.0], [float("inf"), 1.0], []):
        p = js.QuantizationParams.from_constant_array(d, js.PER_TENSOR_SYMMETRIC)
        s, zp = orc.from_constant_array(np.array(d, np.float64))
        assert p.scale == s and p.zero_point == zp


@pytest.mark.parametrize("shape,axis", [((12, 40), 0), ((12, 40), 1), ((3, 5, 7), 1), ((64, 16), 1)])
def test_per_channel_weights_agree(orc, shape, axis):
    rng = np.random.default_rng(3)
    w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    w.reshape(-1)[5] = np.nan
    if axis == 1 and len(shape) == 2:
        w[:, 2] = 0.125                                                  # a constant channel
    flat = f32_list(w)
    p = js.QuantizationParams.from_constant_array_per_channel(flat, list(shape), axis)
    sc = orc.per_channel_scales(w, shape, axis)
    assert (np.array(p.scale).view(np.uint64) == sc.view(np.uint64)).all()
    codes = p.quantize_array_per_channel(flat, list(shape))               # per_channel scheme: clamp [-128, 127]
    q8, qd = orc.quantize_per_channel(w, shape, axis, sc, want_double=True)
    jd = np.array(codes, np.float64).reshape(shape)
    assert ((jd == qd) | (np.isnan(jd) & np.isnan(qd))).all()
    assert (np.array([js.to_int8(c) for c in codes], np.int8).reshape(shape) == q8).all()
    deq = p.dequantize_array_per_channel([float(v) for v in q8.reshape(-1)], list(shape))
    assert (np.array(deq).reshape(shape) == orc.dequantize_per_channel(q8, shape, axis, sc)).all()


# --------------------------------------------------------------------------------------------------- mode C (compiled ops)
@pytest.mark.parametrize("scale,zp,target", [(6 / 127, 0, "i8"), (0.02, 3, "i8"), (1e-3, -5, "i8"), (12 / 255, 128, "ui8"), (0.05, 0, "ui8"),
                                             (6 / 127, -128, "i8"), (3.0, 0, "i8")])
def test_compiled_quantize_dequantize_agree(orc, scale, zp, target):
    rng = np.random.default_rng(int(scale * 1e6) + zp)
    n = 150000                                                               # seven parameter sets: over 10^6 values in all
    x = (rng.standard_normal(n) * 3).astype(np.float32)
    ties = []
    for k in range(-130, 260):
        ties += neighbours(js.fround((k + 0.5 - zp) * scale))
    special = [float("nan"), float("inf"), float("-inf"), 0.0, -0.0, 1e30, -1e30, 1e-45, 3.4e38]
    x = np.concatenate([x, np.array(ties + special, np.float32)])
    dt = 1 if target == "ui8" else 0
    q = orc.quantize_static(x, scale, zp, dt)
    jq = [js.compiled_quantize(v, scale, zp, target) for v in f32_list(x)]
    assert (np.array(jq, q.dtype) == q).all()
    y = orc.dequantize_static(q, scale, zp)
    jy = [js.compiled_dequantize(int(v), scale, zp) for v in q]
    assert (bits32(jy) == y.view(np.uint32)).all()
    acc = rng.integers(-2 ** 31, 2 ** 31, size=2000).astype(np.int32)         # the i32 form (result of quantized_dot)
    y = orc.dequantize_static(acc, scale * 1e-4, zp)
    jy = [js.compiled_dequantize(int(v), scale * 1e-4, zp) for v in acc]
    assert (bits32(jy) == y.view(np.uint32)).all()


# --------------------------------------------------------------------------------------------------- contraction and tail
def test_quantized_dot_agrees(orc):
    rng = np.random.default_rng(4)
    A = rng.integers(-128, 128, size=(9, 70)).astype(np.int8)
    W = rng.integers(-128, 128, size=(11, 70)).astype(np.int8)
    for zpa, zpb in ((0, 0), (3, -5), (-128, 127)):
        ref = orc.qdot_i32(A, W, "NK", zpa, zpb)
        got = js.quantized_dot(A.tolist(), W.tolist(), zpa, zpb)
        assert (np.array(got, np.int32) == ref).all()


@pytest.mark.parametrize("act", ["none", "relu", "gelu_sigmoid", "silu", "gelu_tanh"])
def test_tail_agrees_on_random_and_extreme_accumulators(orc, act):
    rng = np.random.default_rng(6)
    M, N = 400, 512                                                           # 2 * 10^5 elements per activation
    acc = rng.integers(-2 ** 20, 2 ** 20, size=(M, N)).astype(np.int32)
    acc[:20] = rng.integers(-2 ** 31, 2 ** 31, size=(20, N))                  # beyond 2^24: the int -> f32 product is not exact in binary32
    a = rng.uniform(0.005, 0.05, M).astype(np.float32)
    a[20:30] = rng.uniform(1e-3, 50.0, 10).astype(np.float32)                  # pre-activations far into both tails of the sigmoid
    w = rng.uniform(1e-3, 1e-2, N).astype(np.float32)
    b = (rng.standard_normal(N) * 0.01).astype(np.float32)
    b[7] = np.nan
    b[9] = np.inf
    b[11] = -np.inf
    ref = orc.epilogue(acc, a, w, b, act)
    got = js.tail(acc.tolist(), f32_list(a), f32_list(w), f32_list(b), act)
    assert same_f32(got, ref)
    ref = orc.epilogue(acc[:8], a[:8], w, None, act)                          # no bias
    got = js.tail(acc[:8].tolist(), f32_list(a[:8]), f32_list(w), None, act)
    assert same_f32(got, ref)
    sv = (a[0].astype(np.float64) * w.astype(np.float64)).astype(np.float32)  # static form: the scale vector as the pass stores it
    ref = orc.epilogue_sv(acc[:8], sv, b, act)
    got = js.tail_sv(acc[:8].tolist(), f32_list(sv), f32_list(b), act)
    assert same_f32(got, ref)


@pytest.mark.parametrize("act", ["relu", "gelu_sigmoid", "silu", "gelu_tanh"])
def test_activation_argument_sweep_agrees(orc, act):
    """Runs of neighbouring binary32 arguments around zero, the points where exp leaves the binary32 range, and a coarse
    sweep of the whole range, non-finite values included."""
    pts = [0.0, -0.0, 1e-45, -1e-45, 88.72283935546875, -88.72283935546875, 103.97, -103.97, 52.0, -52.0, 17.0, -17.0, 1.0, -1.0, 709.0, -709.0]
    vals = []
    for p in pts:
        vals += neighbours(p, 40)
        vals += neighbours(js.fround(p / 1.702), 40)
    vals += [float(v) for v in np.linspace(-120, 120, 20001).astype(np.float32)]
    vals += [float("nan"), float("inf"), float("-inf"), 3e38, -3e38]
    y = np.array(vals, np.float32)
    ref = orc.activation(y, act)
    got = [js.activation(v, act) for v in f32_list(y)]
    assert same_f32(got, ref)


# --------------------------------------------------------------------------------------------------- f32 block pieces
def test_layer_norm_and_attention_agree(orc):
    rng = np.random.default_rng(8)
    M, D = 6, 96
    x = rng.standard_normal((M, D)).astype(np.float32)
    r = rng.standard_normal((M, D)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    b = (0.1 * rng.standard_normal(D)).astype(np.float32)
    y, s = orc.layer_norm(x, g, b, 1e-5, add=r, want_sum=True)
    jy, jsum = js.layer_norm([f32_list(v) for v in x], f32_list(g), f32_list(b), 1e-5, add=[f32_list(v) for v in r])
    assert (bits32(jy).reshape(M, D) == y.view(np.uint32)).all() and (bits32(jsum).reshape(M, D) == s.view(np.uint32)).all()
    B, H, S, Dh = 2, 2, 9, 64
    q, k, v = (rng.standard_normal((B * S, H * Dh)).astype(np.float32) for _ in range(3))
    for causal in (True, False):
        ref = orc.sdpa(q, k, v, B, H, S, Dh, 0.125, causal)
        got = js.sdpa([f32_list(t) for t in q], [f32_list(t) for t in k], [f32_list(t) for t in v], B, H, S, Dh, 0.125, causal)
        assert (bits32(got).reshape(ref.shape) == ref.view(np.uint32)).all()


def test_mulberry32_agrees(orc):
    nxt = js.make_rng(12345)
    assert [nxt() for _ in range(100)] == list(orc.rng_uniform(12345, 100))


# ------------------------------------------------------------------ per-group codes and the int8 convolution
@pytest.mark.parametrize("n,G,bits", [(4096, 32, 4), (1000, 128, 4), (777, 16, 3), (513, 64, 8), (64, 7, 2)])
def test_per_group_matches(orc, n, G, bits):
    rng = np.random.default_rng(n + G)
    x = (rng.standard_normal(n) * np.exp(rng.uniform(-3, 3, n))).astype(np.float32)
    x[3] = np.nan; x[G:2 * G] = 0.0; x[2 * G + 1] = np.inf; x[5 * G:6 * G] = -2.5      # NaN, an all-zero group, an infinite scale, a constant group
    x[7 * G % n] = np.float32(1e-42)
    qp = js.QuantizationParams.from_constant_array_per_group(f32_list(x), G, "i8", bits)
    s = orc.per_group_scales(x, G, bits)
    assert list(s) == qp.scale
    q8, qd = orc.quantize_per_group(x, G, s, bits, want_double=True)
    q_js = qp.quantize_array_per_group(f32_list(x))
    assert all((a == b) or (a != a and b != b) for a, b in zip(qd, q_js))
    assert list(q8) == [js.to_int8(v) for v in q_js]
    d = orc.dequantize_per_group(q8, G, s)
    d_js = qp.dequantize_array_per_group([int(v) for v in q8])
    assert all((a == b) or (a != a and b != b) for a, b in zip(d, d_js))


CONV_CASES = [
    # N, C, H, W, O, KH, KW, strides, padding, dilation, groups, zp_in, zp_ker
    (2, 4, 7, 6, 6, 3, 3, (2, 1), ((1, 0), (2, 1)), (1, 2), 2, 3, -2),
    (1, 3, 8, 8, 5, 3, 3, (1, 1), ((1, 1), (1, 1)), (1, 1), 1, 0, 0),
    (2, 16, 5, 5, 8, 1, 1, (1, 1), ((0, 0), (0, 0)), (1, 1), 1, 0, 0),
    (1, 6, 9, 7, 6, 2, 3, (2, 2), ((0, 1), (1, 0)), (2, 1), 6, -5, 7),
    (1, 2, 4, 4, 2, 4, 4, (1, 1), ((3, 3), (3, 3)), (1, 1), 1, 127, -128),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_quantized_conv_matches(orc, case):
    N, C, H, W, O, KH, KW, st, pad, dil, groups, zi, zk = case
    rng = np.random.default_rng(N * 100 + C)
    x = rng.integers(-128, 128, (N, C, H, W), dtype=np.int8)
    k = rng.integers(-128, 128, (O, C // groups, KH, KW), dtype=np.int8)
    ref = js.quantized_conv2d(x.tolist(), k.tolist(), st, pad, dil, groups, zi, zk)
    got = orc.quantized_conv2d(x, k, st, pad, dil, groups, zi, zk, "NCHW")
    assert np.array_equal(got, np.array(ref, np.int32))
    # the channel-last form is the same numbers re-laid
    got_l = orc.quantized_conv2d(np.ascontiguousarray(x.transpose(0, 2, 3, 1)), np.ascontiguousarray(k.transpose(0, 2, 3, 1)),
                                 st, pad, dil, groups, zi, zk, "NHWC")
    assert np.array_equal(got_l.transpose(0, 3, 1, 2), got)
