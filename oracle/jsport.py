"""A second, independent restatement of the reference's CPU arithmetic for the quantized-linear path, in pure Python.

TEST INFRASTRUCTURE ONLY: nothing in the product may import this module (``tests/``, the golden-fixture generator and
nothing else use it).  Its purpose is to pin the C++ oracle (``oracle.cpp``): the two were written separately from
the same TypeScript sources, one line of Python per line of TypeScript here, and ``tests/test_jsport_vs_oracle.py``
demands that they agree bit for bit on millions of values and on every constructed edge case.  The committed golden
fixtures (``tests/golden/*.npz``) are generated from THIS module, not from the C++ oracle.

Why pure Python: a Python ``float`` is an IEEE binary64 number, exactly what a JavaScript ``number`` is, and ``+ - * /``
on it round the same way, so JavaScript expressions carry over symbol for symbol.  ``Math.fround`` goes through
``struct`` (binary32 and back), ``Math.round`` / ``|0`` / typed-array stores are written out from the ECMAScript
rules.  No numpy arithmetic is on any path below (numpy only packs results for the callers).  ``Math.exp`` /
``Math.tanh`` are taken from ``math`` (the C library's, as in the C++ oracle): the one thing the two restatements
share, and the one thing that can differ from V8's own routines in the last place.

Paths cited are inside the reference project (slexisvn/mlfw v0.1.6).
"""
from __future__ import annotations

import math
import struct

NAN = float("nan")
INF = float("inf")


# ---------------------------------------------------------------------------------------------- ECMAScript numbers
def math_round(x: float) -> float:
    """Math.round: the integer nearest to x, ties toward +Infinity; NaN and the infinities pass through."""
    if x != x or x in (INF, -INF):
        return x
    r = math.floor(x)
    return float(r + 1) if x - r >= 0.5 else float(r)


def fround(v: float) -> float:
    """Math.fround: round to binary32 (nearest, ties to even), return as a number."""
    if v != v or v in (INF, -INF):
        return v
    try:
        return struct.unpack("<f", struct.pack("<f", v))[0]
    except OverflowError:          # beyond the binary32 range: rounds to an infinity (struct refuses instead)
        return INF if v > 0 else -INF


def math_max(a: float, b: float) -> float:
    """Math.max of two numbers: NaN if either is NaN."""
    if a != a or b != b:
        return NAN
    return a if a > b else b


def math_min(a: float, b: float) -> float:
    if a != a or b != b:
        return NAN
    return a if a < b else b


def to_int32(v: float) -> int:
    """ToInt32 (the `|0` of a cast to an integer dtype): NaN and the infinities give 0, otherwise truncate and wrap."""
    if v != v or v in (INF, -INF):
        return 0
    t = int(v)                     # truncates toward zero
    t &= 0xFFFFFFFF
    return t - (1 << 32) if t & 0x80000000 else t


def to_int8(v: float) -> int:
    """Store into an Int8Array."""
    t = to_int32(v) & 0xFF
    return t - 256 if t & 0x80 else t


def to_uint8(v: float) -> int:
    return to_int32(v) & 0xFF


def js_or(x: float, fallback: float) -> float:
    """x || fallback for numbers: 0, -0 and NaN are falsy."""
    return fallback if (x == 0.0 or x != x) else x


# ------------------------------------------------------------- QuantizationParams (src/compiler/ir/graph/quantization_types.ts)
PER_TENSOR_SYMMETRIC, PER_TENSOR_ASYMMETRIC, PER_CHANNEL = "per_tensor_symmetric", "per_tensor_asymmetric", "per_channel"
PER_GROUP = "per_group"


class QuantizationParams:
    """quantization_types.ts:41-141.  `scale` / `zero_point` are numbers, or lists for the per-channel scheme."""

    def __init__(self, scheme, scale, zero_point, axis=None, dtype="i8", num_bits=8, group_size=None):
        self.scheme, self.scale, self.zero_point, self.axis, self.dtype, self.num_bits = scheme, scale, zero_point, axis, dtype, num_bits
        self.group_size = group_size

    def is_symmetric(self):
        return self.scheme == PER_TENSOR_SYMMETRIC

    def clamp_range(self):                                   # :62-73
        if self.is_symmetric():
            bound = 2 ** (self.num_bits - 1) - 1
            return [-bound, bound]
        if self.dtype == "ui8":
            return [0, 2 ** self.num_bits - 1]
        return [-(2 ** (self.num_bits - 1)), 2 ** (self.num_bits - 1) - 1]

    def quantize(self, float_val):                           # :75-79
        c_min, c_max = self.clamp_range()
        raw = math_round(_div(float_val, self.scale) + self.zero_point)
        return math_max(c_min, math_min(c_max, raw))

    def dequantize(self, int_val):                           # :81-83
        return (int_val - self.zero_point) * self.scale

    def quantize_array(self, arr):                           # :85-97
        c_min, c_max = self.clamp_range()
        s, zp = self.scale, self.zero_point
        return [math_max(c_min, math_min(c_max, math_round(_div(v, s) + zp))) for v in arr]

    def dequantize_array(self, arr):                         # :99-110
        s, zp = self.scale, self.zero_point
        return [(q - zp) * s for q in arr]

    def _channel_stride(self, shape):                        # :112-116
        stride = 1
        for d in range(self.axis + 1, len(shape)):
            stride *= shape[d]
        return stride

    def quantize_array_per_channel(self, arr, shape):        # :118-130
        c_min, c_max = self.clamp_range()
        stride = self._channel_stride(shape)
        num_ch = shape[self.axis]
        out = [0.0] * len(arr)
        for i in range(len(arr)):
            ch = (i // stride) % num_ch
            s, zp = self.scale[ch], self.zero_point[ch]
            out[i] = math_max(c_min, math_min(c_max, math_round(_div(arr[i], s) + zp)))
        return out

    def dequantize_array_per_channel(self, arr, shape):      # :132-141
        stride = self._channel_stride(shape)
        num_ch = shape[self.axis]
        return [(arr[i] - self.zero_point[(i // stride) % num_ch]) * self.scale[(i // stride) % num_ch] for i in range(len(arr))]

    def quantize_array_per_group(self, arr):                 # :143-153
        c_min, c_max = self.clamp_range()
        out = [0.0] * len(arr)
        for i in range(len(arr)):
            g = i // self.group_size
            s, zp = self.scale[g], self.zero_point[g]
            out[i] = math_max(c_min, math_min(c_max, math_round(_div(arr[i], s) + zp)))
        return out

    def dequantize_array_per_group(self, arr):               # :155-162
        return [(arr[i] - self.zero_point[i // self.group_size]) * self.scale[i // self.group_size] for i in range(len(arr))]

    # ---- factories
    @staticmethod
    def from_range(mn, mx, scheme, dtype="i8", num_bits=8):  # :248-264
        if scheme == PER_TENSOR_SYMMETRIC:
            abs_max = max(abs(mn), abs(mx)) if not (mn != mn or mx != mx) else NAN
            bound = 2 ** (num_bits - 1) - 1
            scale = js_or(abs_max / bound, 1e-10)
            return QuantizationParams(scheme, scale, 0, None, dtype, num_bits)
        c_min, c_max = (0, 2 ** num_bits - 1) if dtype == "ui8" else (-(2 ** (num_bits - 1)), 2 ** (num_bits - 1) - 1)
        rng = js_or(mx - mn, 1e-10)
        scale = rng / (c_max - c_min)
        zero_point = math_round(c_min - _div(mn, scale))
        clamped = math_max(c_min, math_min(c_max, zero_point))
        return QuantizationParams(scheme, scale, clamped, None, dtype, num_bits)

    @staticmethod
    def from_range_per_channel(mins, maxs, axis, dtype="i8", num_bits=8):   # :266-281
        bound = 2 ** (num_bits - 1) - 1
        scales = []
        for c in range(len(mins)):
            abs_max = max(abs(mins[c]), abs(maxs[c]))
            scales.append(js_or(abs_max / bound, 1e-10))
        return QuantizationParams(PER_CHANNEL, scales, [0] * len(mins), axis, dtype, num_bits)

    @staticmethod
    def default_for_activation(scheme, dtype="i8", num_bits=8):             # :283-285
        return QuantizationParams.from_range(-6, 6, scheme, dtype, num_bits)

    @staticmethod
    def from_constant_array(data, scheme, dtype="i8", num_bits=8):          # :287-297
        mn, mx = INF, -INF
        for v in data:
            if v < mn:
                mn = v
            if v > mx:
                mx = v
        if not math.isfinite(mn):
            mn = -1
        if not math.isfinite(mx):
            mx = 1
        if mn == mx:
            mn -= 0.5
            mx += 0.5
        return QuantizationParams.from_range(mn, mx, scheme, dtype, num_bits)

    @staticmethod
    def from_constant_array_per_channel(data, shape, axis, dtype="i8", num_bits=8):   # :299-317
        num_ch = shape[axis]
        stride = 1
        for d in range(axis + 1, len(shape)):
            stride *= shape[d]
        mins, maxs = [INF] * num_ch, [-INF] * num_ch
        for i in range(len(data)):
            ch = (i // stride) % num_ch
            v = data[i]
            if v < mins[ch]:
                mins[ch] = v
            if v > maxs[ch]:
                maxs[ch] = v
        for c in range(num_ch):
            if not math.isfinite(mins[c]):
                mins[c] = -1
            if not math.isfinite(maxs[c]):
                maxs[c] = 1
            if mins[c] == maxs[c]:
                mins[c] -= 0.5
                maxs[c] += 0.5
        return QuantizationParams.from_range_per_channel(mins, maxs, axis, dtype, num_bits)

    @staticmethod
    def from_constant_array_per_group(data, group_size, dtype="i8", num_bits=4):      # :319-340
        num_groups = -(-len(data) // group_size)
        scales, zero_points = [0.0] * num_groups, [0] * num_groups
        bound = 2 ** (num_bits - 1) - 1
        for g in range(num_groups):
            start = g * group_size
            end = min(start + group_size, len(data))
            abs_max = 0.0
            for i in range(start, end):
                a = abs(data[i])
                if a > abs_max:
                    abs_max = a
            scales[g] = js_or(abs_max / bound, 1e-10)
        return QuantizationParams(PER_GROUP, scales, zero_points, None, dtype, num_bits, group_size)


def _div(a: float, b: float) -> float:
    """JavaScript division: a zero divisor gives an infinity or NaN instead of raising."""
    try:
        return a / b
    except ZeroDivisionError:
        if a != a or a == 0:
            return NAN
        neg = (math.copysign(1.0, a) < 0) != (math.copysign(1.0, b) < 0)
        return -INF if neg else INF


# ------------------------------------------------------------------------------ per-token = per-channel along axis 0
def quantize_per_token(rows, c_min=-127.0, c_max=127.0):
    """`rows`: list of rows of binary32 values.  Returns (codes as stored in an Int8Array, binary64 scales, scales rounded
    to binary32).  fromConstantArrayPerChannel(x, [M, K], 0) + quantizeArrayPerChannel; the clamp is passed in because the
    device interface takes it as a parameter (with absmax scaling [-127, 127] and [-128, 127] give the same codes)."""
    M, K = len(rows), len(rows[0]) if rows else 0
    flat = [v for r in rows for v in r]
    qp = QuantizationParams.from_constant_array_per_channel(flat, [M, K], 0)
    codes = []
    for i, v in enumerate(flat):
        s = qp.scale[(i // K) % M]
        codes.append(to_int8(math_max(c_min, math_min(c_max, math_round(_div(v, s) + 0)))))
    return [codes[m * K:(m + 1) * K] for m in range(M)], list(qp.scale), [fround(s) for s in qp.scale]


def dequantize_per_token_f32(codes, scales32):
    """(q - 0) * scale with the binary32 scales the device interface carries, stored to a Float32Array."""
    return [[fround((q - 0) * s) for q in row] for row, s in zip(codes, scales32)]


# ------------------------------------------- compiled ops (src/compiler/passes/lowering/quant_math.ts:16-34 as emitted by
# src/backend/cpu/codegen.ts:474-545: every f32 binary op is `Math.fround(a op b)`, round/max/min are exact externs,
# the cast to an integer dtype is `(v | 0)` and the store into the typed array truncates once more)
def compiled_quantize(x: float, scale: float, zero_point: int = 0, target: str = "i8") -> int:
    c_min, c_max = (0, 255) if target == "ui8" else (-128, 127)
    t = fround(_div(x, scale))
    if zero_point != 0:
        t = fround(t + zero_point)
    r = math_round(t)
    c = math_min(math_max(r, c_min), c_max)
    v = to_int32(c)
    return (v & 0xFF) if target == "ui8" else to_int8(v)


def compiled_dequantize(q: int, scale: float, zero_point: int = 0) -> float:
    v = float(q)                       # (+q): the cast to f32 of an integer is not rounded
    if zero_point != 0:
        v = fround(v - zero_point)
    return fround(v * scale)


# ------------------------------------------------------ quantized_dot (src/compiler/passes/lowering/rules/quantization.ts:23-42)
def quantized_dot(A, W_nk, zp_a=0, zp_b=0):
    """C[m][n] = sum_k ((A|0) - zpA) * ((B|0) - zpB), accumulated as numbers, stored to an Int32Array."""
    out = []
    for a in A:
        row = []
        for w in W_nk:
            acc = 0
            for x, y in zip(a, w):
                acc = acc + (x - zp_a) * (y - zp_b)
            row.append(to_int32(float(acc)))
        out.append(row)
    return out


# ------------------------------------------------------ quantized_conv (src/compiler/passes/lowering/rules/quantization.ts:44-62
# over the loop nest of lowering_registry.ts:335-449; output extents ops/linalg.ts:236-246)
def quantized_conv2d(x, ker, strides=(1, 1), padding=((0, 0), (0, 0)), dilation=(1, 1), groups=1, zp_in=0, zp_ker=0):
    """x: nested lists [N][C][H][W] of int8 codes, ker: [O][C/groups][KH][KW]; returns [N][O][OH][OW] as stored to an
    Int32Array.  The loops run in the nest's order (n, oc, oh, ow, ic, kh, kw); a tap outside the input adds the guard's 0."""
    N, C, H, W = len(x), len(x[0]), len(x[0][0]), len(x[0][0][0])
    O, Cg, KH, KW = len(ker), len(ker[0]), len(ker[0][0]), len(ker[0][0][0])
    OH = math.floor((H + padding[0][0] + padding[0][1] - ((KH - 1) * dilation[0] + 1)) / strides[0]) + 1
    OW = math.floor((W + padding[1][0] + padding[1][1] - ((KW - 1) * dilation[1] + 1)) / strides[1]) + 1
    group_size = O // groups
    out = [[[[0] * OW for _ in range(OH)] for _ in range(O)] for _ in range(N)]
    for n in range(N):
        for oc in range(O):
            for oh in range(OH):
                for ow in range(OW):
                    acc = 0
                    for ic in range(Cg):
                        c = (oc // group_size) * Cg + ic if groups > 1 else ic
                        for kh in range(KH):
                            for kw in range(KW):
                                ih = oh * strides[0] + (kh * dilation[0] + -padding[0][0])
                                iw = ow * strides[1] + (kw * dilation[1] + -padding[1][0])
                                inside = 1
                                if padding[0][0] != 0 or padding[0][1] != 0:
                                    inside *= (1 if ih >= 0 else 0) * (1 if ih < H else 0)
                                if padding[1][0] != 0 or padding[1][1] != 0:
                                    inside *= (1 if iw >= 0 else 0) * (1 if iw < W else 0)
                                prod = (x[n][c][ih][iw] - zp_in) * (ker[oc][ic][kh][kw] - zp_ker) if inside else 0
                                acc = to_int32(float(acc + prod))
                    out[n][oc][oh][ow] = acc
    return out


# ------------------------------- tail (quantization_pass.ts:427-456, nn/functional/linear.ts:13-15, decomposition_pass.ts:197-230)
def sigmoid(z: float) -> float:
    """emitSigmoid on the CPU target: neg is exact, exp rounds once, 1 + e rounds, 1 / d rounds."""
    e = fround(math.exp(-z)) if -z < 709.0 else INF
    d = fround(1.0 + e)
    return fround(_div(1.0, d))


def activation(y: float, act: str) -> float:
    if act == "none":
        return y
    if act == "relu":                                  # maximum(x, broadcast 0) -> Math.max
        return math_max(y, 0.0)
    if act == "gelu_sigmoid":                          # x * sigmoid(1.702 x), 1.702 a binary64 immediate
        z = fround(1.702 * y)
        return fround(y * sigmoid(z))
    if act == "silu":
        return fround(y * sigmoid(y))
    if act == "gelu_tanh":                             # no reference form: the standard one, every binary op rounded
        y2 = fround(y * y)
        y3 = fround(y2 * y)
        c = fround(0.044715 * y3)
        inner = fround(y + c)
        u = fround(0.7978845608028654 * inner)
        t = fround(math.tanh(u))
        o = fround(1.0 + t)
        h = fround(0.5 * y)
        return fround(h * o)
    raise ValueError(act)


def tail(acc, a_scales32, w_scales32, bias32, act: str):
    """convert -> mul(scale vector) -> add(bias) -> activation: sv = fround(aScale * wScale[n]) (a product of two numbers
    stored as an f32 constant), t = fround((+acc) * sv), y = fround(t + bias[n]).  `a_scales32` has one entry per row."""
    out = []
    for m, row in enumerate(acc):
        o = []
        for n, a in enumerate(row):
            sv = fround(a_scales32[m] * w_scales32[n])
            t = fround(float(a) * sv)
            y = fround(t + bias32[n]) if bias32 is not None else t
            o.append(activation(y, act))
        out.append(o)
    return out


def tail_sv(acc, sv32, bias32, act: str):
    """The same tail when the scale vector is given (static activation scale folded in by the pass)."""
    return [[activation(fround(fround(float(a) * sv32[n]) + bias32[n]) if bias32 is not None else fround(float(a) * sv32[n]), act)
             for n, a in enumerate(row)] for row in acc]


# --------------------------------------------------------------------- f32 pieces of the block, index-order binary32
def layer_norm(rows, gamma, beta, eps, add=None):
    """decomposition_pass.ts:232-260, every operation rounded to binary32, reductions in index order.  Returns (y, sum)."""
    D = len(gamma)
    eps32 = fround(eps)
    ys, sums = [], []
    for m, r in enumerate(rows):
        row = [fround(v + add[m][d]) if add is not None else v for d, v in enumerate(r)]
        sums.append(list(row))
        acc = 0.0
        for v in row:
            acc = fround(acc + v)
        mean = fround(acc / D)
        acc2 = 0.0
        cen = []
        for v in row:
            c = fround(v - mean)
            cen.append(c)
            acc2 = fround(acc2 + fround(c * c))
        var = fround(acc2 / D)
        ve = fround(var + eps32)
        rstd = fround(1.0 / math.sqrt(ve))
        ys.append([fround(fround(fround(c * rstd) * gamma[d]) + beta[d]) for d, c in enumerate(cen)])
    return ys, sums


def sdpa(q, k, v, B, H, S, Dh, scale, causal=True):
    """src/nn/functional/attention.ts:42-74 with the softmax of decomposition_pass.ts:156-174; rows are (b, s), the
    columns of head h start at h * Dh.  Every operation rounded to binary32, sums in index order."""
    scale32 = fround(scale)
    out = [[0.0] * (H * Dh) for _ in range(B * S)]
    for b in range(B):
        for h in range(H):
            for i in range(S):
                qi = q[b * S + i][h * Dh:(h + 1) * Dh]
                sc = []
                mx = -INF
                for j in range(S):
                    kj = k[b * S + j][h * Dh:(h + 1) * Dh]
                    acc = 0.0
                    for d in range(Dh):
                        acc = fround(acc + fround(qi[d] * kj[d]))
                    s = fround(acc * scale32)
                    if causal:
                        s = fround(s + (0.0 if j <= i else -INF))
                    sc.append(s)
                    if s > mx:
                        mx = s
                total = 0.0
                for j in range(S):
                    e = fround(math.exp(fround(sc[j] - mx)))
                    sc[j] = e
                    total = fround(total + e)
                for d in range(Dh):
                    acc = 0.0
                    for j in range(S):
                        w = fround(sc[j] / total)
                        acc = fround(acc + fround(w * v[b * S + j][h * Dh + d]))
                    out[b * S + i][h * Dh + d] = acc
    return out


# ------------------------------------------------- calibration observers (src/compiler/analysis/calibration.ts:11-186)
class HistogramCollector:
    def __init__(self, num_bins=2048):
        self.num_bins, self.bins = num_bins, [0.0] * num_bins
        self.range_min = self.range_max = 0.0
        self.initialized, self.total_count = False, 0

    def update(self, data):                                   # :57-79
        if not self.initialized:
            self._init_range(data)
        rng = self.range_max - self.range_min
        if not rng > 0:
            return
        for v in data:
            if v < self.range_min or v > self.range_max:
                self._expand_and_rebucket(data)
                return
        scale = _div(self.num_bins, rng)
        for v in data:
            self._bump((v - self.range_min) * scale)
        self.total_count += len(data)

    def _bump(self, raw, by=1.0):
        """bins[Math.min(numBins - 1, Math.floor(raw))] += by; an index that is not a number stores nowhere."""
        if raw != raw:
            return
        f = raw if raw in (INF, -INF) else float(math.floor(raw))
        idx = math_min(self.num_bins - 1, f)
        if idx == idx and idx >= 0:
            self.bins[int(idx)] += by

    def _init_range(self, data):                              # :81-90
        mn, mx = INF, -INF
        for v in data:
            if v < mn:
                mn = v
            if v > mx:
                mx = v
        if mn == mx:
            mx = mn + 1
        self.range_min, self.range_max, self.initialized = mn, mx, True

    def _expand_and_rebucket(self, new_data):                 # :92-120
        new_min, new_max = self.range_min, self.range_max
        for v in new_data:
            if v < new_min:
                new_min = v
            if v > new_max:
                new_max = v
        old_bins, old_min, old_range = list(self.bins), self.range_min, self.range_max - self.range_min
        self.range_min, self.range_max = new_min, new_max
        new_scale = _div(self.num_bins, new_max - new_min)
        self.bins = [0.0] * self.num_bins
        if old_range > 0:
            width = old_range / self.num_bins
            for i in range(self.num_bins):
                if old_bins[i] == 0:
                    continue
                center = old_min + (i + 0.5) * width
                self._bump((center - new_min) * new_scale, old_bins[i])
        for v in new_data:
            self._bump((v - new_min) * new_scale)
        self.total_count += len(new_data)

    def compute_percentile_threshold(self, percentile):       # :130-141
        target = self.total_count * percentile
        cumulative = 0.0
        width = (self.range_max - self.range_min) / self.num_bins
        for i in range(self.num_bins):
            cumulative += self.bins[i]
            if cumulative >= target:
                return self.range_min + (i + 1) * width
        return self.range_max

    def compute_entropy_threshold(self, num_quant_bins):      # :143-186
        if self.total_count == 0:
            return self.range_max
        ref = [b / self.total_count for b in self.bins]
        best_idx, best_kl = self.num_bins, INF
        for t in range(num_quant_bins, self.num_bins + 1):
            qw = t / num_quant_bins
            q = [0.0] * t
            for i in range(num_quant_bins):
                start = math.floor(i * qw)
                end = min(t, math.floor((i + 1) * qw))
                total = 0.0
                for j in range(start, end):
                    total += ref[j]
                if end - start > 0:
                    avg = total / (end - start)
                    for j in range(start, end):
                        q[j] = avg
            kl = 0.0
            for i in range(t):
                if ref[i] > 0 and q[i] > 0:
                    kl += ref[i] * math.log(ref[i] / q[i])
            if kl < best_kl:
                best_kl, best_idx = kl, t
        width = (self.range_max - self.range_min) / self.num_bins
        return self.range_min + best_idx * width


# ----------------------------------------------------------------------------------------------------- seeded data
def make_rng(seed: int):
    """mulberry32, src/util/random.ts:5-14."""
    state = [seed & 0xFFFFFFFF]

    def imul(a, b):
        return (a * b) & 0xFFFFFFFF

    def nxt():
        state[0] = (state[0] + 0x6D2B79F5) & 0xFFFFFFFF
        a = state[0]
        t = imul(a ^ (a >> 15), 1 | a)
        t = ((t + imul(t ^ (t >> 7), 61 | t)) & 0xFFFFFFFF) ^ t
        return ((t ^ (t >> 14)) & 0xFFFFFFFF) / 4294967296.0
    return nxt
