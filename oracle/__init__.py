"""ctypes front end of the CPU oracle (``oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU-baseline leg of ``bench.py``.  The product package never imports it.

Every function here forwards to the C++ restatement, which cites the reference
file and line it follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

SCHEME_SYM, SCHEME_ASYM, SCHEME_PER_CHANNEL = 0, 1, 2
DT_I8, DT_UI8 = 0, 1
ACT = {"none": 0, "relu": 1, "gelu_sigmoid": 2, "gelu_tanh": 3, "silu": 4}


def build(force: bool = False) -> str:
    """Compile ``oracle.cpp`` with the Makefile beside it; returns the library path."""
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "liboracle.so"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_qp_quantize.restype = C.c_double
        _lib.orc_qp_quantize.argtypes = [C.c_double] * 5
        _lib.orc_qp_dequantize.restype = C.c_double
        _lib.orc_qp_dequantize.argtypes = [C.c_double] * 3
        _lib.orc_js_round.restype = C.c_double
        _lib.orc_js_round.argtypes = [C.c_double]
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ----------------------------------------------------------------- seeded data
def rng_uniform(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, np.float64)
    lib().orc_rng_uniform(C.c_uint32(seed & 0xFFFFFFFF), C.c_int64(n), _p(out))
    return out


def normal_f32(seed: int, shape, mean=0.0, std=1.0) -> np.ndarray:
    out = np.empty(int(np.prod(shape)), np.float32)
    lib().orc_normal_f32(C.c_uint32(seed & 0xFFFFFFFF), C.c_int64(out.size), C.c_double(mean), C.c_double(std), _p(out))
    return out.reshape(shape)


def uniform_f32(seed: int, shape, a=0.0, b=1.0) -> np.ndarray:
    out = np.empty(int(np.prod(shape)), np.float32)
    lib().orc_uniform_f32(C.c_uint32(seed & 0xFFFFFFFF), C.c_int64(out.size), C.c_double(a), C.c_double(b), _p(out))
    return out.reshape(shape)


def randint_i8(seed: int, shape, lo=-127, hi=127) -> np.ndarray:
    out = np.empty(int(np.prod(shape)), np.int8)
    lib().orc_randint_i8(C.c_uint32(seed & 0xFFFFFFFF), C.c_int64(out.size), C.c_int(lo), C.c_int(hi), _p(out))
    return out.reshape(shape)


# --------------------------------------------------------- QuantizationParams
def clamp_range(scheme=SCHEME_SYM, dtype=DT_I8, num_bits=8):
    a, b = C.c_double(), C.c_double()
    lib().orc_qp_clamp_range(C.c_int(scheme), C.c_int(dtype), C.c_int(num_bits), C.byref(a), C.byref(b))
    return a.value, b.value


def from_range(mn, mx, scheme=SCHEME_SYM, dtype=DT_I8, num_bits=8):
    s, z = C.c_double(), C.c_double()
    lib().orc_qp_from_range(C.c_double(mn), C.c_double(mx), C.c_int(scheme), C.c_int(dtype), C.c_int(num_bits),
                            C.byref(s), C.byref(z))
    return s.value, z.value


def from_constant_array(data, scheme=SCHEME_SYM, dtype=DT_I8, num_bits=8):
    d = np.ascontiguousarray(data, np.float64)
    s, z = C.c_double(), C.c_double()
    lib().orc_qp_from_constant_array(_p(d), C.c_int64(d.size), C.c_int(scheme), C.c_int(dtype), C.c_int(num_bits),
                                     C.byref(s), C.byref(z))
    return s.value, z.value


def qp_quantize(x, scale, zp, cmin, cmax) -> float:
    return lib().orc_qp_quantize(x, scale, zp, cmin, cmax)


def qp_dequantize(q, scale, zp) -> float:
    return lib().orc_qp_dequantize(q, scale, zp)


def js_round(x: float) -> float:
    return lib().orc_js_round(x)


def _axis_view(shape, axis):
    shape = tuple(int(s) for s in shape)
    outer = int(np.prod(shape[:axis])) if axis > 0 else 1
    stride = int(np.prod(shape[axis + 1:])) if axis + 1 < len(shape) else 1
    return outer, shape[axis], stride


def per_channel_scales(data, shape, axis, num_bits=8) -> np.ndarray:
    outer, nch, stride = _axis_view(shape, axis)
    scales = np.empty(nch, np.float64)
    if np.asarray(data).dtype == np.float32:
        d = _f32(data)
        lib().orc_per_channel_scales_f32(_p(d), C.c_int64(outer), C.c_int64(nch), C.c_int64(stride), C.c_int(num_bits), _p(scales))
    else:
        d = np.ascontiguousarray(data, np.float64)
        lib().orc_per_channel_scales_f64(_p(d), C.c_int64(outer), C.c_int64(nch), C.c_int64(stride), C.c_int(num_bits), _p(scales))
    return scales


def quantize_per_channel(data, shape, axis, scales, cmin=-128.0, cmax=127.0, want_double=False):
    """Returns int8 codes (as stored to an Int8Array) and, optionally, the raw double codes."""
    outer, nch, stride = _axis_view(shape, axis)
    scales = np.ascontiguousarray(scales, np.float64)
    n = outer * nch * stride
    q8 = np.empty(n, np.int8)
    qd = np.empty(n, np.float64) if want_double else None
    if np.asarray(data).dtype == np.float32:
        d = _f32(data)
        fn = lib().orc_quantize_per_channel_f32
    else:
        d = np.ascontiguousarray(data, np.float64)
        fn = lib().orc_quantize_per_channel_f64
    fn(_p(d), C.c_int64(outer), C.c_int64(nch), C.c_int64(stride), _p(scales), C.c_double(cmin), C.c_double(cmax), _p(q8), _p(qd))
    q8 = q8.reshape(shape)
    return (q8, qd.reshape(shape)) if want_double else q8


def dequantize_per_channel(q, shape, axis, scales) -> np.ndarray:
    outer, nch, stride = _axis_view(shape, axis)
    q = np.ascontiguousarray(q, np.int8)
    scales = np.ascontiguousarray(scales, np.float64)
    out = np.empty(q.size, np.float64)
    lib().orc_dequantize_per_channel(_p(q), C.c_int64(outer), C.c_int64(nch), C.c_int64(stride), _p(scales), _p(out))
    return out.reshape(shape)


def per_group_scales(data, group_size, num_bits=4) -> np.ndarray:
    """QuantizationParams.fromConstantArrayPerGroup (quantization_types.ts:319-340): one binary64 scale per run of
    ``group_size`` consecutive elements of the flat array."""
    flat = np.asarray(data).reshape(-1)
    n = flat.size
    scales = np.empty((n + group_size - 1) // group_size, np.float64)
    if flat.dtype == np.float32:
        d = _f32(flat)
        lib().orc_per_group_scales_f32(_p(d), C.c_int64(n), C.c_int64(group_size), C.c_int(num_bits), _p(scales))
    else:
        d = np.ascontiguousarray(flat, np.float64)
        lib().orc_per_group_scales_f64(_p(d), C.c_int64(n), C.c_int64(group_size), C.c_int(num_bits), _p(scales))
    return scales


def quantize_per_group(data, group_size, scales, num_bits=4, want_double=False):
    """quantizeArrayPerGroup (quantization_types.ts:143-153): codes as stored to an Int8Array, optionally the raw doubles."""
    flat = np.asarray(data).reshape(-1)
    n = flat.size
    scales = np.ascontiguousarray(scales, np.float64)
    q8 = np.empty(n, np.int8)
    qd = np.empty(n, np.float64) if want_double else None
    if flat.dtype == np.float32:
        d, fn = _f32(flat), lib().orc_quantize_per_group_f32
    else:
        d, fn = np.ascontiguousarray(flat, np.float64), lib().orc_quantize_per_group_f64
    fn(_p(d), C.c_int64(n), C.c_int64(group_size), C.c_int(num_bits), _p(scales), _p(q8), _p(qd))
    return (q8, qd) if want_double else q8


def dequantize_per_group(q, group_size, scales) -> np.ndarray:
    """dequantizeArrayPerGroup (quantization_types.ts:155-162), binary64 result."""
    q = np.ascontiguousarray(np.asarray(q).reshape(-1), np.int8)
    scales = np.ascontiguousarray(scales, np.float64)
    out = np.empty(q.size, np.float64)
    lib().orc_dequantize_per_group(_p(q), C.c_int64(q.size), C.c_int64(group_size), _p(scales), _p(out))
    return out


def conv_out_extent(size, pad_lo, pad_hi, k, stride, dilation) -> int:
    """ops/linalg.ts:236-246."""
    return (size + pad_lo + pad_hi - ((k - 1) * dilation + 1)) // stride + 1


def quantized_conv2d(x, ker, strides=(1, 1), padding=((0, 0), (0, 0)), dilation=(1, 1), groups=1, zp_in=0, zp_ker=0,
                     layout="NCHW") -> np.ndarray:
    """quantized_conv (lowering rules/quantization.ts:44-62): int8 input [N,C,H,W] x int8 kernel [O,C/groups,KH,KW]
    -> int32 [N,O,OH,OW]; with layout "NHWC": [N,H,W,C] x [O,KH,KW,C/groups] -> [N,OH,OW,O]."""
    x = np.ascontiguousarray(x, np.int8)
    ker = np.ascontiguousarray(ker, np.int8)
    lay = {"NCHW": 0, "NHWC": 1}[layout]
    if lay == 0:
        N, Cc, H, W = x.shape
        O, _, KH, KW = ker.shape
    else:
        N, H, W, Cc = x.shape
        O, KH, KW, _ = ker.shape
    OH = conv_out_extent(H, padding[0][0], padding[0][1], KH, strides[0], dilation[0])
    OW = conv_out_extent(W, padding[1][0], padding[1][1], KW, strides[1], dilation[1])
    out = np.empty((N, O, OH, OW) if lay == 0 else (N, OH, OW, O), np.int32)
    lib().orc_quantized_conv2d(_p(x), _p(ker), C.c_int64(N), C.c_int64(Cc), C.c_int64(H), C.c_int64(W), C.c_int64(O),
                               C.c_int64(KH), C.c_int64(KW), C.c_int(strides[0]), C.c_int(strides[1]),
                               C.c_int(padding[0][0]), C.c_int(padding[0][1]), C.c_int(padding[1][0]), C.c_int(padding[1][1]),
                               C.c_int(dilation[0]), C.c_int(dilation[1]), C.c_int(groups), C.c_int(zp_in), C.c_int(zp_ker),
                               C.c_int(lay), _p(out))
    return out


def quantize_per_token(x, cmin=-127.0, cmax=127.0):
    """Per-token (row) symmetric int8: returns (codes int8 [M,K], scales f64 [M], scales f32 [M])."""
    x = _f32(x)
    M, K = x.shape
    q = np.empty((M, K), np.int8)
    s64 = np.empty(M, np.float64)
    s32 = np.empty(M, np.float32)
    lib().orc_quantize_per_token(_p(x), C.c_int64(M), C.c_int64(K), C.c_double(cmin), C.c_double(cmax), _p(q), _p(s64), _p(s32))
    return q, s64, s32


def dequantize_per_token_f32(q, scales32) -> np.ndarray:
    q = np.ascontiguousarray(q, np.int8)
    s = _f32(scales32)
    M, K = q.shape
    y = np.empty((M, K), np.float32)
    lib().orc_dequantize_per_token_f32(_p(q), _p(s), C.c_int64(M), C.c_int64(K), _p(y))
    return y


# ------------------------------------------------------ compiled ops (mode C)
def quantize_static(x, scale, zp=0, dtype=DT_I8) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.int8)
    lib().orc_quantize_static(_p(x), C.c_int64(x.size), C.c_double(scale), C.c_double(zp), C.c_int(dtype), _p(out))
    return out.view(np.uint8) if dtype == DT_UI8 else out


def dequantize_static(q, scale, zp=0) -> np.ndarray:
    q = np.ascontiguousarray(q)
    y = np.empty(q.shape, np.float32)
    fn = {np.dtype(np.int8): "orc_dequantize_static_i8", np.dtype(np.uint8): "orc_dequantize_static_u8",
          np.dtype(np.int32): "orc_dequantize_static_i32"}[q.dtype]
    getattr(lib(), fn)(_p(q), C.c_int64(q.size), C.c_double(scale), C.c_double(zp), _p(y))
    return y


def qdot_i32(A, W, w_layout="NK", zpA=0, zpB=0, threads=0) -> np.ndarray:
    """A int8 [M,K]; W int8 [N,K] (layout 'NK') or [K,N] ('KN'); returns int32 [M,N]."""
    A = np.ascontiguousarray(A, np.int8)
    W = np.ascontiguousarray(W, np.int8)
    M, K = A.shape
    N = W.shape[0] if w_layout == "NK" else W.shape[1]
    assert (W.shape[1] if w_layout == "NK" else W.shape[0]) == K
    out = np.empty((M, N), np.int32)
    lib().orc_qdot_i32(_p(A), _p(W), C.c_int64(M), C.c_int64(N), C.c_int64(K), C.c_int(0 if w_layout == "NK" else 1),
                       C.c_int(zpA), C.c_int(zpB), _p(out), C.c_int(threads))
    return out


def epilogue(acc, a_scales, w_scales, bias=None, act="none") -> np.ndarray:
    """Per-channel tail + bias + activation; a_scales is a scalar (static) or an [M] array (per token)."""
    acc = np.ascontiguousarray(acc, np.int32)
    M, N = acc.shape
    a = _f32(np.atleast_1d(a_scales))
    per_token = int(a.size == M and np.ndim(a_scales) > 0)
    w = _f32(w_scales)
    b = _f32(bias) if bias is not None else None
    out = np.empty((M, N), np.float32)
    lib().orc_epilogue(_p(acc), C.c_int64(M), C.c_int64(N), _p(a), C.c_int(per_token), _p(w), _p(b), C.c_int(ACT[act]), _p(out))
    return out


def epilogue_sv(acc, sv, bias=None, act="none") -> np.ndarray:
    acc = np.ascontiguousarray(acc, np.int32)
    M, N = acc.shape
    sv = _f32(sv)
    b = _f32(bias) if bias is not None else None
    out = np.empty((M, N), np.float32)
    lib().orc_epilogue_sv(_p(acc), C.c_int64(M), C.c_int64(N), _p(sv), _p(b), C.c_int(ACT[act]), _p(out))
    return out


def activation(y, act) -> np.ndarray:
    y = _f32(y)
    out = np.empty(y.shape, np.float32)
    lib().orc_activation(_p(y), C.c_int64(y.size), C.c_int(ACT[act]), _p(out))
    return out


def layer_norm(x, gamma, beta, eps=1e-5, add=None, want_sum=False):
    """LayerNorm over the last axis of x [M, D] (+ add first); returns y (and x + add when want_sum)."""
    x = _f32(x)
    M, D = x.shape
    a = _f32(add) if add is not None else None
    y = np.empty((M, D), np.float32)
    s = np.empty((M, D), np.float32) if want_sum else None
    lib().orc_layer_norm(_p(x), _p(a), _p(_f32(gamma)), _p(_f32(beta)), C.c_double(eps), C.c_int64(M), C.c_int64(D), _p(s), _p(y))
    return (y, s) if want_sum else y


def sdpa(q, k, v, B, H, S, Dh, scale, causal=True, rows=None):
    """Attention over q, k, v given as [B*S, H*Dh] arrays (row (b, s), columns of head h at h*Dh).  Returns the same
    layout, or, with ``rows`` (flattened (b*H + h)*S + i indices), a dense [len(rows), Dh] array of just those rows."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    ld = H * Dh
    assert q.shape == (B * S, ld) and k.shape == q.shape and v.shape == q.shape
    if rows is None:
        out = np.zeros((B * S, ld), np.float32)
        lib().orc_sdpa(_p(q), _p(k), _p(v), C.c_int64(ld), C.c_int64(ld), C.c_int64(ld), C.c_int64(B), C.c_int64(H), C.c_int64(S),
                       C.c_int64(Dh), C.c_double(scale), C.c_int(int(causal)), None, C.c_int64(0), _p(out), C.c_int64(ld))
        return out
    r = np.ascontiguousarray(rows, np.int64)
    out = np.zeros((r.size, Dh), np.float32)
    lib().orc_sdpa(_p(q), _p(k), _p(v), C.c_int64(ld), C.c_int64(ld), C.c_int64(ld), C.c_int64(B), C.c_int64(H), C.c_int64(S),
                   C.c_int64(Dh), C.c_double(scale), C.c_int(int(causal)), _p(r), C.c_int64(r.size), _p(out), C.c_int64(Dh))
    return out


def minmax_observe(batches):
    mn, mx = C.c_double(float("inf")), C.c_double(float("-inf"))
    for b in batches:
        b = _f32(b)
        lib().orc_minmax_observe(_p(b), C.c_int64(b.size), C.byref(mn), C.byref(mx))
    return mn.value, mx.value


def num_threads() -> int:
    return lib().orc_num_threads()


def set_num_threads(n: int) -> None:
    """Threads of the OpenMP loops from now on (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    lib().orc_set_num_threads(C.c_int(int(n)))


def usable_cores() -> int:
    import os
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def linear(x, wq, w_scales, bias=None, act="none", w_layout="NK", threads=0):
    """f32 activations -> per-token quantize -> int32 GEMM -> per-channel tail: the whole hot path."""
    q, _, s32 = quantize_per_token(x)
    acc = qdot_i32(q, wq, w_layout, threads=threads)
    return epilogue(acc, s32, w_scales, bias, act), q, s32, acc
