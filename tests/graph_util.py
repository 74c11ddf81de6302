"""Builds, for the tests, the graphs the reference's QuantizationPass emits (flat: fusion disabled on the target).

``quantized_linear`` follows QuantizationPass._replacePerChannelDot (src/compiler/passes/quantization/
quantization_pass.ts:390-459) op for op; the bias add and the activation follow nn/functional/linear.ts:13-15,
builder.ts:561-565 and decomposition_pass.ts:197-230.  Weight scales and codes come from the CPU oracle.
"""
import numpy as np

from mlfw_b200.backend import GraphBuilder


def quantized_linear(b: GraphBuilder, orc, x, w, bias, a_scale, act="none", w_is_kn=True):
    """x: Value f32 [..., K]; w: f32 array [K,N] (w_is_kn) or [N,K]; returns the result Value and a dict of facts."""
    w = np.asarray(w, np.float32)
    K, N = (w.shape if w_is_kn else w.shape[::-1])
    channel_axis = 1 if w_is_kn else 0
    wsc = orc.per_channel_scales(w, w.shape, channel_axis)                       # binary64, one per output channel
    wq = orc.quantize_per_channel(w, w.shape, channel_axis, wsc, -128, 127)
    wc = b.constant(wq.reshape(-1).tolist(), w.shape, "i8")
    xq = b.op("quantize", [x], x.shape, "i8", scale=a_scale, zero_point=0, scheme="per_tensor_symmetric", target_dtype="i8")
    out_shape = tuple(x.shape[:-1]) + (N,)
    qd = b.op("quantized_dot", [xq, wc], out_shape, "i32", lhs_contracting=[len(x.shape) - 1],
              rhs_contracting=[0 if w_is_kn else 1], lhs_scale=a_scale, lhs_zero_point=0, rhs_scale=1, rhs_zero_point=0,
              output_scale=1, output_zero_point=0)
    cf = b.op("convert", [qd], out_shape, "f32", target_dtype="f32")
    scale_vec = [a_scale * float(s) for s in wsc]                                # binary64 products, as in the pass
    sv = b.constant(scale_vec, (N,), "f32")
    bc = b.op("broadcast_in_dim", [sv], out_shape, "f32", broadcast_dimensions=[len(out_shape) - 1], result_shape=list(out_shape))
    y = b.op("mul", [cf, bc], out_shape, "f32")
    if bias is not None:
        bcst = b.constant(np.asarray(bias, np.float64).tolist(), (N,), "f32")
        bb = b.op("broadcast_in_dim", [bcst], out_shape, "f32", broadcast_dimensions=[len(out_shape) - 1], result_shape=list(out_shape))
        y = b.op("add", [y, bb], out_shape, "f32")
    y = activation(b, y, act)
    return y, {"wq": wq, "wsc": wsc, "scale_vec": np.array(scale_vec), "K": K, "N": N, "w_is_kn": w_is_kn}


def _bcast_scalar(b, value, shape):
    c = b.constant(value, (), "f32")
    return b.op("broadcast_in_dim", [c], shape, "f32", broadcast_dimensions=[], result_shape=list(shape))


def sigmoid(b, x):
    neg = b.op("neg", [x], x.shape, "f32")
    e = b.op("exp", [neg], x.shape, "f32")
    one = _bcast_scalar(b, 1, x.shape)
    den = b.op("add", [one, e], x.shape, "f32")
    return b.op("div", [one, den], x.shape, "f32")


def activation(b, y, act):
    if act == "none":
        return y
    if act == "relu":
        return b.op("maximum", [y, _bcast_scalar(b, 0, y.shape)], y.shape, "f32")
    if act == "silu":
        return b.op("mul", [y, sigmoid(b, y)], y.shape, "f32")
    if act == "gelu_sigmoid":
        scaled = b.op("mul", [_bcast_scalar(b, 1.702, y.shape), y], y.shape, "f32")
        return b.op("mul", [y, sigmoid(b, scaled)], y.shape, "f32")
    raise ValueError(act)
