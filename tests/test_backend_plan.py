"""CPU tests of the host-side mirror: the planner recognises the graph contract and rejects everything else."""
import numpy as np
import pytest

from graph_util import activation, quantized_linear
from mlfw_b200.backend import (B200CompileError, B200Target, GraphBuilder, TARGET_ATTR_EXTERNAL_COMPILER,
                               TARGET_ATTR_FUSION, compile_with_b200, plan_function, program_of, steps_from_program)


def mlp_graph(orc, act="relu", w_is_kn=True, M=8, K=32, H=64, N=16):
    rng = np.random.default_rng(0)
    w1 = rng.standard_normal((K, H) if w_is_kn else (H, K)).astype(np.float32) * 0.1
    w2 = rng.standard_normal((H, N) if w_is_kn else (N, H)).astype(np.float32) * 0.1
    b1 = rng.uniform(-0.1, 0.1, H).astype(np.float32)
    b2 = rng.uniform(-0.1, 0.1, N).astype(np.float32)
    b = GraphBuilder("mlp")
    x = b.arg((M, K))
    h, f1 = quantized_linear(b, orc, x, w1, b1, 6 / 127, act, w_is_kn)
    y, f2 = quantized_linear(b, orc, h, w2, b2, 4 / 127, "none", w_is_kn)
    return b.ret(y), (f1, f2, b1, b2)


def test_target_object():
    t = B200Target()
    assert t["kind"] == "accelerator" and t["supportsInt8"] and t["attrs"][TARGET_ATTR_FUSION] == {"enabled": False}
    assert t["attrs"][TARGET_ATTR_EXTERNAL_COMPILER] is compile_with_b200
    with pytest.raises(ValueError):
        B200Target(activationQuant="bogus")


@pytest.mark.parametrize("act", ["none", "relu", "silu", "gelu_sigmoid"])
@pytest.mark.parametrize("w_is_kn", [True, False])
def test_static_plan_fuses_tail_and_next_quantize(orc, act, w_is_kn):
    func, (f1, f2, b1, b2) = mlp_graph(orc, act, w_is_kn)
    steps = plan_function(func, dynamic=False)
    assert [s.kind for s in steps] == ["quantize_static", "linear", "linear"]
    l1, l2 = steps[1].params, steps[2].params
    assert (l1["M"], l1["K"], l1["N"], l1["act"]) == (8, 32, 64, act)
    assert l1["requant_scale"] == 4 / 127 and l2["requant_scale"] is None      # layer 2's quantize rides in layer 1's epilogue
    assert (l1["w_scales"] == f1["scale_vec"].astype(np.float32)).all()         # the graph's f32 scale-vector constant
    assert (l1["bias"] == b1).all() and (l2["bias"] == b2).all()
    assert (l1["w"] == f1["wq"]).all() and l1["w_layout"] == (1 if w_is_kn else 0)
    assert steps[2].out is func.returns[0]


def test_dynamic_plan_recovers_weight_scales(orc):
    func, (f1, f2, _, _) = mlp_graph(orc, "relu")
    steps = plan_function(func, dynamic=True)
    assert [s.kind for s in steps] == ["quantize_token", "linear", "quantize_token", "linear"]
    assert steps[1].params["a_dynamic"] and steps[1].params["requant_scale"] is None
    np.testing.assert_array_equal(steps[1].params["w_scales"], (f1["scale_vec"] / (6 / 127)).astype(np.float32))
    assert np.abs(steps[1].params["w_scales"] / f1["wsc"] - 1).max() < 1e-6


def test_standalone_quantize_dequantize(orc):
    b = GraphBuilder("rt")
    x = b.arg((6,))
    q = b.op("quantize", [x], (6,), "i8", scale=6 / 127, zero_point=0, target_dtype="i8")
    y = b.op("dequantize", [q], (6,), "f32", scale=6 / 127, zero_point=0)
    steps = plan_function(b.ret(y), dynamic=False)
    assert [s.kind for s in steps] == ["quantize_static", "dequantize_static"]


def test_per_tensor_path(orc):
    """quantize, quantize(const) folded, quantized_dot, dequantize(scale = lhs*rhs) (quantization_pass.ts:286-360)."""
    b = GraphBuilder("pt")
    x = b.arg((4, 8))
    wq = np.arange(-24, 24, dtype=np.int8).reshape(8, 6)
    xq = b.op("quantize", [x], (4, 8), "i8", scale=0.05, zero_point=0, target_dtype="i8")
    wc = b.constant(wq.reshape(-1).tolist(), (8, 6), "i8")
    qd = b.op("quantized_dot", [xq, wc], (4, 6), "i32", lhs_contracting=[1], rhs_contracting=[0], lhs_scale=0.05, rhs_scale=0.02,
              output_scale=0.001)
    y = b.op("dequantize", [qd], (4, 6), "f32", scale=0.05 * 0.02, zero_point=0)
    steps = plan_function(b.ret(y), dynamic=False)
    # the compiled `dequantize` multiplies by a binary64 immediate: the contraction and the tail are steps of their own
    assert [s.kind for s in steps] == ["quantize_static", "dot", "tail"]
    assert steps[2].params["tensor_scale"] == 0.05 * 0.02 and steps[2].params["w_scales"] is None and steps[2].ins[0] is steps[1].out


def test_ops_outside_the_contract_are_refused(orc):
    b = GraphBuilder("bad")
    x = b.arg((4, 8))
    y = b.op("softmax", [x], (4, 8), "f32")
    with pytest.raises(B200CompileError, match="outside the graph contract"):
        plan_function(b.ret(y), dynamic=False)
    b = GraphBuilder("bad2")
    x = b.arg((4, 8))
    xq = b.op("quantize", [x], (4, 8), "i8", scale=0.05, zero_point=0)
    w = b.arg((8, 6), "i8")                                  # non-constant weights
    qd = b.op("quantized_dot", [xq, w], (4, 6), "i32", lhs_contracting=[1], rhs_contracting=[0])
    with pytest.raises(B200CompileError, match="constant rank-2 int8"):
        plan_function(b.ret(qd), dynamic=False)
    b = GraphBuilder("bad3")                                 # fake-quant boundary around an elementwise op (D10)
    x = b.arg((4,))
    q = b.op("quantize", [x], (4,), "i8", scale=0.05, zero_point=0)
    d = b.op("dequantize", [q], (4,), "f32", scale=0.05, zero_point=0)
    a = b.op("add", [d, d], (4,), "f32")
    with pytest.raises(B200CompileError, match="'add'"):
        plan_function(b.ret(a), dynamic=False)


def test_rank3_lhs_flattens_to_rows(orc):
    rng = np.random.default_rng(1)
    b = GraphBuilder("r3")
    x = b.arg((2, 5, 16))
    y, _ = quantized_linear(b, orc, x, rng.standard_normal((24, 16)).astype(np.float32), None, 0.03, "none", w_is_kn=False)
    steps = plan_function(b.ret(y), dynamic=True)
    assert steps[0].params["M"] == 10 and steps[1].params["M"] == 10 and steps[1].params["N"] == 24


@pytest.mark.parametrize("dynamic", [False, True])
def test_native_program_round_trips_through_json(orc, dynamic):
    """The planned function as data (the `source` of a serialized kernel): through JSON and back it yields the same
    steps, shapes, parameters and constant arrays, wired to the same values."""
    import json
    func, _ = mlp_graph(orc, "gelu_sigmoid", w_is_kn=False)
    steps = plan_function(func, dynamic=dynamic)
    text = json.dumps(program_of(func.args, func.returns, steps))
    args, returns, again = steps_from_program(json.loads(text))
    assert [(a.shape, a.dtype) for a in args] == [(a.shape, a.dtype) for a in func.args]
    assert len(again) == len(steps) and len(returns) == 1 and returns[0] is again[-1].out
    for a, b in zip(steps, again):
        assert a.kind == b.kind and a.out.shape == b.out.shape and a.out.dtype == b.out.dtype
        assert set(a.params) == set(b.params)
        for k, v in a.params.items():
            if isinstance(v, np.ndarray):
                assert b.params[k].dtype == v.dtype and b.params[k].shape == v.shape and (b.params[k] == v).all()
            else:
                assert b.params[k] == v
    # the data flow survives: every step after the first reads what an earlier step (or an argument) produced
    produced = {id(v) for v in args}
    for st in again:
        assert all(id(v) in produced for v in st.ins)
        produced.add(id(st.out))


def test_native_program_rejects_what_it_does_not_understand(orc):
    func, _ = mlp_graph(orc)
    prog = program_of(func.args, func.returns, plan_function(func, dynamic=False))
    with pytest.raises(B200CompileError, match="version"):
        steps_from_program({**prog, "version": 99})
    bad = {**prog, "steps": [{**prog["steps"][0], "kind": "pooling"}] + prog["steps"][1:]}
    with pytest.raises(B200CompileError, match="unknown step"):
        steps_from_program(bad)
    with pytest.raises(B200CompileError, match="never produced"):
        steps_from_program({**prog, "returns": [12345]})


def conv_graph(orc, layout="NCHW"):
    """The reference pass's conv pipeline (tests/compiler/passes/quantization/pass.test.js:428-440):
    quantize(input), quantize(kernel), quantized_conv, dequantize."""
    rng = np.random.default_rng(3)
    N, C, H, W, O, KH, KW = 2, 4, 9, 8, 6, 3, 3
    k = (rng.standard_normal((O, C // 2, KH, KW)) * 0.2).astype(np.float32)
    x_shape = (N, C, H, W)
    if layout == "NHWC":
        k = np.ascontiguousarray(k.transpose(0, 2, 3, 1))
        x_shape = (N, H, W, C)
    in_scale, _ = orc.from_range(-6, 6)
    k_scale, _ = orc.from_constant_array(k.astype(np.float64).reshape(-1))
    b = GraphBuilder("conv")
    x = b.arg(x_shape)
    xq = b.op("quantize", [x], x_shape, "i8", scale=in_scale, zero_point=0, target_dtype="i8")
    kc = b.constant(k.tolist(), k.shape, "f32")
    kq = b.op("quantize", [kc], k.shape, "i8", scale=k_scale, zero_point=0, target_dtype="i8")
    OH, OW = orc.conv_out_extent(H, 1, 1, KH, 2, 1), orc.conv_out_extent(W, 0, 2, KW, 1, 1)
    out_shape = (N, O, OH, OW) if layout == "NCHW" else (N, OH, OW, O)
    acc = b.op("quantized_conv", [xq, kq], out_shape, "i32", strides=[2, 1], padding=[[1, 1], [0, 2]], dilation=[1, 1], groups=2,
               input_layout=layout, kernel_layout="OIHW" if layout == "NCHW" else "OHWI", input_scale=in_scale, input_zero_point=0,
               kernel_scale=k_scale, kernel_zero_point=0, output_scale=in_scale * k_scale, output_zero_point=0)
    y = b.op("dequantize", [acc], out_shape, "f32", scale=in_scale * k_scale, zero_point=0)
    return b.ret(y), {"k": k, "in_scale": in_scale, "k_scale": k_scale, "x_shape": x_shape, "out_shape": out_shape}


@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
def test_conv_pipeline_plans_and_round_trips(orc, layout):
    import json
    func, info = conv_graph(orc, layout)
    steps = plan_function(func, dynamic=False)
    assert [s.kind for s in steps] == ["quantize_static", "const", "quantize_static", "conv", "dequantize_static"]
    assert steps[1].params["data"].dtype == np.float32 and (steps[1].params["data"] == info["k"]).all()
    conv = steps[3]
    assert conv.params["shape"] == [2, 4, 9, 8] and conv.params["kernel_shape"] == [6, 3, 3] and conv.params["groups"] == 2
    assert conv.params["layout"] == layout and conv.out.dtype == "i32" and conv.out.shape == info["out_shape"]
    args, returns, again = steps_from_program(json.loads(json.dumps(program_of(func.args, func.returns, steps))))
    assert [s.kind for s in again] == [s.kind for s in steps]
    assert again[1].params["data"].dtype == np.float32 and (again[1].params["data"] == info["k"]).all()
    assert again[3].params == conv.params and again[3].ins[1] is again[2].out and returns[0] is again[4].out


def test_conv_outside_the_contract_is_refused(orc):
    b = GraphBuilder("c")
    x = b.arg((1, 2, 4, 4), "ui8")
    k = b.arg((2, 2, 1, 1), "i8")
    y = b.op("quantized_conv", [x, k], (1, 2, 4, 4), "i32", strides=[1, 1], padding=[[0, 0], [0, 0]], input_layout="NCHW", kernel_layout="OIHW")
    steps = plan_function(b.ret(y), dynamic=False)       # ui8 input: shifted by 128, zero-point moved along
    assert [s.kind for s in steps] == ["shift", "conv"] and steps[1].params["zp_in"] == -128 and steps[1].ins[0] is steps[0].out
    b = GraphBuilder("c")
    x, k = b.arg((1, 2, 4, 4), "i8"), b.arg((2, 2, 1, 1), "i8")
    y = b.op("quantized_conv", [x, k], (1, 2, 4, 4), "i32", strides=[1, 1], padding=[[0, 0], [0, 0]], input_layout="NCHW", kernel_layout="HWIO")
    with pytest.raises(B200CompileError, match="layouts"):
        plan_function(b.ret(y), dynamic=False)


def asymmetric_graph(orc, M=6, K=32, N=10):
    """The per-tensor asymmetric form: quantize{zero_point}, quantized_dot{lhs_zero_point, rhs_zero_point} on constant
    codes, dequantize{scale = lhs_scale * rhs_scale} (quantization_pass.ts:286-360 with an asymmetric scheme)."""
    rng = np.random.default_rng(8)
    a_scale, a_zp, w_scale, w_zp = 0.04, 7, 0.01, -3
    wq = rng.integers(-128, 128, (K, N), dtype=np.int8)
    b = GraphBuilder("asym")
    x = b.arg((M, K))
    xq = b.op("quantize", [x], (M, K), "i8", scale=a_scale, zero_point=a_zp, scheme="per_tensor_asymmetric", target_dtype="i8")
    wc = b.constant(wq.reshape(-1).tolist(), (K, N), "i8")
    acc = b.op("quantized_dot", [xq, wc], (M, N), "i32", lhs_contracting=[1], rhs_contracting=[0], lhs_scale=a_scale, lhs_zero_point=a_zp,
               rhs_scale=w_scale, rhs_zero_point=w_zp, output_scale=a_scale * w_scale, output_zero_point=0)
    y = b.op("dequantize", [acc], (M, N), "f32", scale=a_scale * w_scale, zero_point=0)
    return b.ret(y), {"wq": wq, "a_scale": a_scale, "a_zp": a_zp, "w_scale": w_scale, "w_zp": w_zp, "M": M, "K": K, "N": N}


def test_zero_point_dot_is_a_step_of_its_own(orc):
    import json
    func, info = asymmetric_graph(orc)
    steps = plan_function(func, dynamic=False)
    assert [s.kind for s in steps] == ["quantize_static", "dot", "tail"]
    assert steps[0].params["zero_point"] == 7 and steps[1].params["zp_a"] == 7 and steps[1].params["zp_w"] == -3
    assert steps[1].out.dtype == "i32" and steps[2].params["tensor_scale"] == 0.04 * 0.01 and steps[2].params["act"] == "none"
    args, returns, again = steps_from_program(json.loads(json.dumps(program_of(func.args, func.returns, steps))))
    assert [s.kind for s in again] == [s.kind for s in steps] and (again[1].params["w"] == info["wq"]).all()


def test_ui8_operands_are_shifted(orc):
    """quantize{ui8, zp} -> quantized_dot{lhs_zero_point} on ui8 constant codes -> dequantize: both operands become int8
    codes 128 lower with zero-points 128 lower (the lhs by a device step, the constant on the host)."""
    rng = np.random.default_rng(2)
    M, K, N = 5, 16, 7
    wq = rng.integers(0, 256, (N, K)).astype(np.uint8)
    b = GraphBuilder("u8")
    x = b.arg((M, K))
    xq = b.op("quantize", [x], (M, K), "ui8", scale=0.03, zero_point=120, target_dtype="ui8")
    wc = b.constant(wq.reshape(-1).tolist(), (N, K), "ui8")
    acc = b.op("quantized_dot", [xq, wc], (M, N), "i32", lhs_contracting=[1], rhs_contracting=[1], lhs_scale=0.03, lhs_zero_point=120,
               rhs_scale=0.01, rhs_zero_point=131)
    y = b.op("dequantize", [acc], (M, N), "f32", scale=0.0003, zero_point=0)
    steps = plan_function(b.ret(y), dynamic=False)
    assert [s.kind for s in steps] == ["quantize_static", "shift", "dot", "tail"]
    dot = steps[2]
    assert dot.params["zp_a"] == -8 and dot.params["zp_w"] == 3 and dot.params["w"].dtype == np.int8
    assert (dot.params["w"].astype(np.int32) == wq.astype(np.int32) - 128).all() and dot.ins[0] is steps[1].out
