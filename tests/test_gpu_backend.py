"""The reference-facing interface end to end on the GPU: graphs as the quantization pass emits them, compiled with
compile_with_b200, run with typed arrays, checked against the CPU oracle's evaluation of the same graph.

test_c1_mlp is benchmark configuration 1: X f32 [256,512] ~ N(0,1), W1 [512,1024], W2 [1024,256] ~ N(0,0.02), biases
~ U(-0.1,0.1), per-output-channel int8 weights, ReLU between the layers, f32 [256,256] out, seed 0."""
import numpy as np
import pytest

from graph_util import quantized_linear
from mlfw_b200 import synth
from mlfw_b200.backend import B200Target, GraphBuilder, compile_with_b200

pytestmark = pytest.mark.gpu


def c1_tensors():
    s = synth.tensor_seed
    x = synth.normal(s(0, 0), (256, 512))
    w1 = synth.normal(s(0, 1), (512, 1024), 0.0, 0.02)
    b1 = synth.uniform(s(0, 2), (1024,), -0.1, 0.1)
    w2 = synth.normal(s(0, 3), (1024, 256), 0.0, 0.02)
    b2 = synth.uniform(s(0, 4), (256,), -0.1, 0.1)
    return x, w1, b1, w2, b2


def build_mlp(orc, x_shape, w1, b1, w2, b2, a1, a2, act="relu"):
    b = GraphBuilder("mlp")
    x = b.arg(x_shape)
    h, f1 = quantized_linear(b, orc, x, w1, b1, a1, act, True)
    y, f2 = quantized_linear(b, orc, h, w2, b2, a2, "none", True)
    return b.ret(y), f1, f2


def test_c1_mlp_static_scales_match_the_reference_chain(orc):
    x, w1, b1, w2, b2 = c1_tensors()
    a1 = orc.from_range(float(x.min()), float(x.max()))[0]          # min/max calibration (calibration.ts:246-268)
    hf = np.maximum(x.astype(np.float64) @ w1 + b1, 0)
    a2 = orc.from_range(float(hf.min()), float(hf.max()))[0]
    func, f1, f2 = build_mlp(orc, x.shape, w1, b1, w2, b2, a1, a2)
    mod = compile_with_b200({"mlp": func}, {"target": B200Target()})
    out = np.zeros((256, 256), np.float32)
    mod.run("mlp", x, out)
    # the same graph as the reference's CPU target evaluates it
    q1 = orc.quantize_static(x, a1)
    h = orc.epilogue_sv(orc.qdot_i32(q1, f1["wq"], "KN"), f1["scale_vec"].astype(np.float32), b1, "relu")
    q2 = orc.quantize_static(h, a2)
    ref = orc.epilogue_sv(orc.qdot_i32(q2, f2["wq"], "KN"), f2["scale_vec"].astype(np.float32), b2, "none")
    assert (out.view(np.uint32) == ref.view(np.uint32)).all()
    # and it is a faithful int8 approximation of the float model (the reference asserts < 3 % for two layers + ReLU)
    yf = hf @ w2 + b2
    assert np.abs(out - yf).sum() / np.abs(yf).sum() < 0.03
    assert mod.listKernels() == ["mlp"] and not mod.isAsync("mlp")
    assert mod.getKernelMetadata("mlp")["steps"] == 3 and "linear" in mod.getKernelSource("mlp")
    # {data, shape, dtype} tensors are accepted as well (tracing/compile.ts:84-95)
    out2 = np.zeros((256, 256), np.float32)
    mod.run("mlp", {"data": x.reshape(-1), "shape": [256, 512], "dtype": "f32"}, {"data": out2, "shape": [256, 256], "dtype": "f32"})
    assert (out2 == out).all()
    with pytest.raises(ValueError, match="takes 1 tensors"):
        mod.run("mlp", x)
    # the serialized module (RuntimeModule.serialize()'s shape, native program as `source`) reloads without the graph
    import json
    from mlfw_b200.backend import B200RuntimeModule
    data = json.loads(json.dumps(mod.serialize()))
    assert data["kernels"][0]["metadata"]["kind"] == "b200" and data["kernels"][0]["target"] == "b200_int8"
    mod.release()
    again = B200RuntimeModule.deserialize(data)
    out3 = np.zeros((256, 256), np.float32)
    again.run("mlp", x, out3)
    assert (out3.view(np.uint32) == ref.view(np.uint32)).all()
    again.release()


def test_c1_mlp_per_token_dynamic(orc):
    x, w1, b1, w2, b2 = c1_tensors()
    func, f1, f2 = build_mlp(orc, x.shape, w1, b1, w2, b2, 6 / 127, 6 / 127)
    mod = compile_with_b200({"mlp": func}, {"target": B200Target(activationQuant="per_token_dynamic")})
    out = np.zeros((256, 256), np.float32)
    mod.run("mlp", x, out)
    ws1 = (f1["scale_vec"] / (6 / 127)).astype(np.float32)
    ws2 = (f2["scale_vec"] / (6 / 127)).astype(np.float32)
    h, q1, s1, acc1 = orc.linear(x, np.ascontiguousarray(f1["wq"].T), ws1, b1, "relu")
    ref, q2, s2, acc2 = orc.linear(h, np.ascontiguousarray(f2["wq"].T), ws2, b2, "none")
    assert (out.view(np.uint32) == ref.view(np.uint32)).all()
    yf = np.maximum(x.astype(np.float64) @ w1 + b1, 0) @ w2 + b2
    assert np.abs(out - yf).sum() / np.abs(yf).sum() < 0.02
    mod.release()


@pytest.mark.parametrize("act", ["silu", "gelu_sigmoid"])
def test_rank3_linear_with_sigmoid_tails(orc, act):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 33, 64)).astype(np.float32)
    w = (rng.standard_normal((96, 64)) * 0.1).astype(np.float32)        # [N,K], a traced Linear
    bias = rng.uniform(-0.1, 0.1, 96).astype(np.float32)
    b = GraphBuilder("lin")
    xv = b.arg(x.shape)
    y, f = quantized_linear(b, orc, xv, w, bias, 0.03, act, w_is_kn=False)
    mod = compile_with_b200({"lin": b.ret(y)}, {"target": B200Target(activationQuant="per_token_dynamic")})
    out = np.zeros((4, 33, 96), np.float32)
    mod.run("lin", x, out)
    ws = (f["scale_vec"] / 0.03).astype(np.float32)
    ref, _, _, _ = orc.linear(x.reshape(-1, 64), f["wq"], ws, bias, act)
    assert (out.reshape(-1, 96).view(np.uint32) == ref.view(np.uint32)).all()
    mod.release()


def test_fake_quant_roundtrip_is_lossy(orc):
    """tests/compiler/passes/quantization/pass.test.js:461-491 on this backend."""
    s, z = orc.from_range(-6, 6)
    data = np.array([3.5, -2.1, 5.9, 1.234, -5.9, 0.001], np.float32)
    b = GraphBuilder("rt")
    x = b.arg((6,))
    q = b.op("quantize", [x], (6,), "i8", scale=s, zero_point=int(z), target_dtype="i8")
    y = b.op("dequantize", [q], (6,), "f32", scale=s, zero_point=int(z))
    mod = compile_with_b200({"rt": b.ret(y)}, {"target": B200Target()})
    out = np.zeros(6, np.float32)
    mod.run("rt", data, out)
    cmin, cmax = orc.clamp_range()
    applied = False
    for i, v in enumerate([3.5, -2.1, 5.9, 1.234, -5.9, 0.001]):
        ref = orc.qp_dequantize(orc.qp_quantize(v, s, z, cmin, cmax), s, z)
        assert abs(out[i] - ref) < 1e-4 and abs(out[i] - v) <= s + 1e-6
        applied |= abs(out[i] - v) > 1e-6
    assert applied
    mod.release()


@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
def test_conv_pipeline_matches_the_reference_chain(orc, layout):
    """quantize(input), quantize(kernel), quantized_conv, dequantize through the target object, and once more from the
    serialized native program; every stage is the CPU oracle's, bit for bit."""
    from test_backend_plan import conv_graph
    from mlfw_b200.backend import B200RuntimeModule
    func, info = conv_graph(orc, layout)
    rng = np.random.default_rng(11)
    x = (rng.standard_normal(info["x_shape"]) * 2.5).astype(np.float32)
    mod = compile_with_b200({"conv": func}, {"target": B200Target()})
    out = np.zeros(info["out_shape"], np.float32)
    mod.run("conv", x, out)
    xq = orc.quantize_static(x.reshape(-1), info["in_scale"]).reshape(x.shape)
    kq = orc.quantize_static(info["k"].reshape(-1), info["k_scale"]).reshape(info["k"].shape)
    acc = orc.quantized_conv2d(xq, kq, (2, 1), ((1, 1), (0, 2)), (1, 1), 2, 0, 0, layout)
    ref = orc.dequantize_static(acc.reshape(-1), info["in_scale"] * info["k_scale"]).reshape(info["out_shape"])
    assert (out.view(np.uint32) == ref.view(np.uint32)).all()
    again = B200RuntimeModule.deserialize(mod.serialize())
    out2 = np.zeros(info["out_shape"], np.float32)
    again.run("conv", x, out2)
    assert (out2.view(np.uint32) == ref.view(np.uint32)).all()
    mod.release(); again.release()


@pytest.mark.parametrize("M,K,N", [(6, 32, 10), (300, 512, 256)])
def test_asymmetric_per_tensor_chain(orc, M, K, N):
    """quantize{zp} -> quantized_dot{zps} -> dequantize through the target object (the larger shape goes through the
    tensor cores plus the zero-point correction terms); every stage is the oracle's."""
    from test_backend_plan import asymmetric_graph
    func, info = asymmetric_graph(orc, M, K, N)
    rng = np.random.default_rng(M)
    x = (rng.standard_normal((M, K)) * 1.5).astype(np.float32)
    mod = compile_with_b200({"asym": func}, {"target": B200Target()})
    out = np.zeros((M, N), np.float32)
    mod.run("asym", x, out)
    xq = orc.quantize_static(x.reshape(-1), info["a_scale"], info["a_zp"]).reshape(M, K)
    acc = orc.qdot_i32(xq, info["wq"], "KN", info["a_zp"], info["w_zp"])
    ref = orc.dequantize_static(acc.reshape(-1), info["a_scale"] * info["w_scale"]).reshape(M, N)
    assert (out.view(np.uint32) == ref.view(np.uint32)).all()
    mod.release()


def test_ui8_operands_through_the_target_object(orc):
    """quantize{ui8, zp} -> quantized_dot on ui8 constant codes -> dequantize: the backend shifts both operands by 128
    (activations on the device, the constant on the host) and moves the zero-points along; sums as plain integer
    arithmetic on the oracle's ui8 codes."""
    rng = np.random.default_rng(21)
    M, K, N = 260, 512, 128
    a_scale, a_zp, w_scale, w_zp = 0.03, 120, 0.01, 131
    wq = rng.integers(0, 256, (N, K)).astype(np.uint8)
    b = GraphBuilder("u8")
    x = b.arg((M, K))
    xq = b.op("quantize", [x], (M, K), "ui8", scale=a_scale, zero_point=a_zp, target_dtype="ui8")
    wc = b.constant(wq.reshape(-1).tolist(), (N, K), "ui8")
    acc = b.op("quantized_dot", [xq, wc], (M, N), "i32", lhs_contracting=[1], rhs_contracting=[1], lhs_scale=a_scale, lhs_zero_point=a_zp,
               rhs_scale=w_scale, rhs_zero_point=w_zp)
    y = b.op("dequantize", [acc], (M, N), "f32", scale=a_scale * w_scale, zero_point=0)
    mod = compile_with_b200({"u8": b.ret(y)}, {"target": B200Target()})
    xv = (rng.standard_normal((M, K)) * 2).astype(np.float32)
    out = np.zeros((M, N), np.float32)
    mod.run("u8", xv, out)
    codes = orc.quantize_static(xv.reshape(-1), a_scale, a_zp, dtype=1).reshape(M, K)
    assert codes.dtype == np.uint8 and codes.min() >= 0 and codes.max() > 127
    sums = ((codes.astype(np.int64) - a_zp) @ (wq.astype(np.int64) - w_zp).T).astype(np.int32)
    ref = orc.dequantize_static(sums.reshape(-1), a_scale * w_scale).reshape(M, N)
    assert (out.view(np.uint32) == ref.view(np.uint32)).all()
    mod.release()


@pytest.mark.parametrize("act", ["none", "relu", "silu"])
def test_per_tensor_path_uses_the_binary64_scale(orc, act):
    """quantize -> quantized_dot -> dequantize{scale} [-> add(bias) -> activation] (quantization_pass.ts:286-360): the
    compiled dequantize is fround((double)acc * scale) with the scale a binary64 immediate; a binary32 scale vector
    would miss that by an ulp on many outputs, so the tail runs as its own kernel with the binary64 scale."""
    from graph_util import activation
    rng = np.random.default_rng(31)
    M, K, N = 200, 256, 96
    a_scale, w_scale = 0.037, 0.0123                    # the product is not a binary32 number
    wq = rng.integers(-127, 128, (K, N), dtype=np.int8)
    bias = rng.standard_normal(N).astype(np.float32)
    b = GraphBuilder("pt")
    x = b.arg((M, K))
    xq = b.op("quantize", [x], (M, K), "i8", scale=a_scale, zero_point=0, target_dtype="i8")
    wc = b.constant(wq.reshape(-1).tolist(), (K, N), "i8")
    acc = b.op("quantized_dot", [xq, wc], (M, N), "i32", lhs_contracting=[1], rhs_contracting=[0], lhs_scale=a_scale, rhs_scale=w_scale)
    y = b.op("dequantize", [acc], (M, N), "f32", scale=a_scale * w_scale, zero_point=0)
    bc = b.constant(bias.astype(np.float64).tolist(), (N,), "f32")
    bb = b.op("broadcast_in_dim", [bc], (M, N), "f32", broadcast_dimensions=[1], result_shape=[M, N])
    y = b.op("add", [y, bb], (M, N), "f32")
    y = activation(b, y, act)
    mod = compile_with_b200({"pt": b.ret(y)}, {"target": B200Target()})
    xv = (rng.standard_normal((M, K)) * 1.5).astype(np.float32)
    out = np.zeros((M, N), np.float32)
    mod.run("pt", xv, out)
    codes = orc.quantize_static(xv.reshape(-1), a_scale).reshape(M, K)
    sums = orc.qdot_i32(codes, wq, "KN")
    deq = orc.dequantize_static(sums.reshape(-1), a_scale * w_scale).reshape(M, N)
    ref = orc.activation((deq + bias).astype(np.float32), act)
    assert (out.view(np.uint32) == ref.view(np.uint32)).all()
    # and the binary32 scale would indeed have differed somewhere
    wrong = (sums.astype(np.float64) * np.float64(np.float32(a_scale * w_scale))).astype(np.float32)
    assert (wrong != deq).any()
    mod.release()
