"""Host-side mirror of the reference's backend interface for this path.

The reference is TypeScript; the image has no JavaScript engine, so the logic a maintainer would add to the
reference (``mlfw_b200/ts/``) is kept here in runnable form with the same names and behaviour:

* :func:`B200Target` — a target description carrying ``EXTERNAL_COMPILER`` (the seam ``TeracTarget`` uses,
  src/backend/terac/target.ts:16-38; consumed at src/compiler/pipeline/compiler.ts:297-329);
* :func:`compile_with_b200` — receives the graph AFTER the reference's graph passes (``QuantizationPass``
  included) and returns a :class:`B200RuntimeModule`;
* :class:`B200RuntimeModule` — ``RuntimeModuleLike`` (src/compiler/support/config_types.ts:58-66): ``run``,
  ``runAsync``, ``isAsync``, ``getKernelSource``, ``getKernelMetadata``, ``listKernels``.

The graph is the reference's graph IR reduced to what matters here: a flat list of ops with the reference's op
names and attributes (fusion is disabled on the target, so no ``fusion`` regions arrive).  Anything outside the
contract raises :class:`B200CompileError` — there is no CPU fallback inside the backend.  This module only plans
and marshals; all arithmetic on tensors happens in ``libb200q.so``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from .device import ACT, Context, KIND, W_KN, W_NK  # noqa: F401


class B200CompileError(RuntimeError):
    pass


# ----------------------------------------------------------------------------- the graph contract
@dataclass(eq=False)
class Value:
    shape: tuple
    dtype: str                      # 'f32', 'i8', 'ui8', 'i32'
    producer: Optional["Op"] = None
    name: str = ""


@dataclass(eq=False)
class Op:
    name: str                       # reference op name: 'quantize', 'quantized_dot', 'convert', 'mul', ...
    operands: List[Value]
    attrs: Dict[str, Any]
    result: Value


@dataclass
class GraphFunction:
    name: str
    args: List[Value]
    ops: List[Op] = field(default_factory=list)
    returns: List[Value] = field(default_factory=list)

    def users(self, v: Value) -> List[Op]:
        return [o for o in self.ops if any(x is v for x in o.operands)]


class GraphBuilder:
    """Builds a :class:`GraphFunction` op by op (the role IRBuilder plays in the reference's tests,
    tests/_utils/ir_fixture.js:10-29)."""

    def __init__(self, name: str):
        self.func = GraphFunction(name, [])

    def arg(self, shape, dtype="f32") -> Value:
        v = Value(tuple(shape), dtype, None, f"arg{len(self.func.args)}")
        self.func.args.append(v)
        return v

    def op(self, name: str, operands: Sequence[Value], shape, dtype: str, **attrs) -> Value:
        res = Value(tuple(shape), dtype)
        o = Op(name, list(operands), dict(attrs), res)
        res.producer = o
        self.func.ops.append(o)
        return res

    def constant(self, value, shape, dtype) -> Value:
        return self.op("constant", [], shape, dtype, value=value)

    def ret(self, *values: Value) -> GraphFunction:
        self.func.returns = list(values)
        return self.func


NP_DTYPE = {"f32": np.float32, "i8": np.int8, "ui8": np.uint8, "i32": np.int32}

TARGET_ATTR_FUSION = "fusion"
TARGET_ATTR_EXTERNAL_COMPILER = "externalCompiler"
B200_OPTIONS = "b200Options"


def B200Target(library: Optional[str] = None, device: int = 0, activationQuant: str = "static") -> dict:
    """The target object a user passes to ``compile(model, inputs, {target: B200Target()})``.

    ``activationQuant='static'`` reproduces the reference's scales (the activation scale the pass baked into the
    graph); ``'per_token_dynamic'`` ignores it, computes one scale per row on the device and recovers the weight
    scales as ``scaleVec[n] / lhs_scale``."""
    if activationQuant not in ("static", "per_token_dynamic"):
        raise ValueError("activationQuant must be 'static' or 'per_token_dynamic'")
    return {
        "kind": "accelerator", "name": "b200_int8", "supportsInt8": True, "supportsConstBuffers": True,
        "attrs": {TARGET_ATTR_FUSION: {"enabled": False}, TARGET_ATTR_EXTERNAL_COMPILER: compile_with_b200,
                  B200_OPTIONS: {"library": library, "device": device, "activationQuant": activationQuant}},
    }


def compile_with_b200(module: Dict[str, GraphFunction], config: dict) -> "B200RuntimeModule":
    """``TargetAttr.EXTERNAL_COMPILER`` hook: ``(GraphModule, CompilerConfig) -> RuntimeModuleLike``."""
    options = config["target"]["attrs"].get(B200_OPTIONS, {})
    return B200RuntimeModule(module, options)


# ----------------------------------------------------------------------------- planning
@dataclass
class Step:
    kind: str                       # 'quantize_static' | 'quantize_token' | 'dequantize_static' | 'linear' | 'dot' | 'tail' | 'conv' | 'const' | 'shift'
    ins: List[Value]
    out: Value
    params: Dict[str, Any]


def _const_array(v: Value) -> Optional[np.ndarray]:
    if v.producer is not None and v.producer.name == "constant":
        val = v.producer.attrs["value"]
        return np.asarray(val, dtype=np.float64).reshape(v.shape if v.shape else ())
    return None


def _broadcast_source(v: Value) -> Optional[Value]:
    """The operand of a broadcast_in_dim / broadcast producing ``v`` (or ``v`` itself if it is a constant)."""
    if v.producer is None:
        return None
    if v.producer.name in ("broadcast_in_dim", "broadcast"):
        return v.producer.operands[0]
    if v.producer.name == "constant":
        return v
    return None


def _scalar_const(v: Value) -> Optional[float]:
    src = _broadcast_source(v)
    if src is None:
        return None
    arr = _const_array(src)
    if arr is None or arr.size != 1:
        return None
    return float(arr.reshape(-1)[0])


class _Planner:
    def __init__(self, func: GraphFunction, dynamic: bool):
        self.f = func
        self.dynamic = dynamic
        self.steps: List[Step] = []
        self.consts: set = set()    # ids of constant values already turned into 'const' steps
        self.done: set = set()      # ids of ops absorbed into a step

    def other(self, op: Op, v: Value) -> Value:
        a, b = op.operands
        return b if a is v else a

    def single_user(self, v: Value, name: str) -> Optional[Op]:
        us = [u for u in self.f.users(v) if id(u) not in self.done]
        return us[0] if len(us) == 1 and us[0].name == name else None

    # ---- activation chains as the decomposition pass emits them (decomposition_pass.ts:197-230, builder.ts:561-565)
    def match_sigmoid(self, z: Value):
        """neg(z) -> exp -> add(1, .) -> div(1, .); returns (result, ops) or None."""
        neg = next((u for u in self.f.users(z) if u.name == "neg"), None)
        if neg is None:
            return None
        exp = self.single_user(neg.result, "exp")
        if exp is None:
            return None
        add = self.single_user(exp.result, "add")
        if add is None or _scalar_const(self.other(add, exp.result)) != 1.0:
            return None
        div = self.single_user(add.result, "div")
        if div is None or div.operands[1] is not add.result or _scalar_const(div.operands[0]) != 1.0:
            return None
        return div.result, [neg, exp, add, div]

    def match_activation(self, y: Value):
        """Returns (act, result value, absorbed ops) for the chain hanging off ``y``; ('none', y, []) if none."""
        users = [u for u in self.f.users(y) if id(u) not in self.done]
        for u in users:
            if u.name == "maximum" and _scalar_const(self.other(u, y)) == 0.0 and len(users) == 1:
                return "relu", u.result, [u]
        # silu: y * sigmoid(y)
        sig = self.match_sigmoid(y)
        if sig is not None:
            res, ops = sig
            mul = next((u for u in self.f.users(res) if u.name == "mul" and any(o is y for o in u.operands)), None)
            if mul is not None:
                return "silu", mul.result, ops + [mul]
        # gelu: y * sigmoid(1.702 * y)
        for u in users:
            if u.name == "mul":
                c = _scalar_const(self.other(u, y))
                if c is not None and abs(c - 1.702) < 1e-12:
                    sig = self.match_sigmoid(u.result)
                    if sig is not None:
                        res, ops = sig
                        mul = next((m for m in self.f.users(res) if m.name == "mul" and any(o is y for o in m.operands)), None)
                        if mul is not None:
                            return "gelu_sigmoid", mul.result, [u] + ops + [mul]
        for u in users:
            if u.name == "gelu_tanh":      # not a reference op: offered for callers that build the graph themselves
                return "gelu_tanh", u.result, [u]
        return "none", y, []

    def plan_dot(self, op: Op):
        lhs, rhs = op.operands
        w = _const_array(rhs)
        if w is None or rhs.dtype not in ("i8", "ui8") or len(rhs.shape) != 2:
            raise B200CompileError("quantized_dot needs a constant rank-2 int8 rhs (weights cross the boundary as buffers)")
        if op.attrs.get("lhs_batch") or op.attrs.get("rhs_batch"):
            raise B200CompileError("batched quantized_dot is not supported: flatten leading dimensions to M")
        rc = list(op.attrs.get("rhs_contracting", [0]))
        lc = list(op.attrs.get("lhs_contracting", [len(lhs.shape) - 1]))
        if lc != [len(lhs.shape) - 1] or len(rc) != 1:
            raise B200CompileError("quantized_dot must contract the last lhs dimension with one rhs dimension")
        w_layout = W_KN if rc[0] == 0 else W_NK
        K = rhs.shape[rc[0]]
        N = rhs.shape[1 - rc[0]]
        M = int(np.prod(lhs.shape[:-1]))      # leading dimensions flatten to rows (cublas_split.ts:84-90 does the same)
        zp_a, zp_w = int(op.attrs.get("lhs_zero_point", 0) or 0), int(op.attrs.get("rhs_zero_point", 0) or 0)
        if rhs.dtype == "ui8":                 # constant ui8 codes: moved by 128 here, on the host
            w, zp_w = w - 128, zp_w - 128
        if lhs.dtype == "ui8":
            zp_a -= 128
        lhs_scale = float(op.attrs.get("lhs_scale", 1.0))
        absorbed = [op]
        y = op.result
        sv = None                              # per-channel scale vector (binary64 numbers of the graph constant)
        tensor_scale = None                    # or the one binary64 scale of a per-tensor `dequantize`
        conv = self.single_user(y, "convert")
        deq = self.single_user(y, "dequantize")
        if conv is not None:                   # per-channel tail: convert -> mul(broadcast(constant f32[N]))
            mul = self.single_user(conv.result, "mul")
            src = _broadcast_source(self.other(mul, conv.result)) if mul is not None else None
            arr = _const_array(src) if src is not None else None
            if mul is None or arr is None or arr.size != N:
                raise B200CompileError("quantized_dot -> convert must be followed by mul with a per-channel scale vector")
            sv = arr.reshape(-1)
            absorbed += [conv, mul]
            y = mul.result
        elif deq is not None:                  # per-tensor path: dequantize(scale = lhs_scale * rhs_scale)
            if deq.attrs.get("zero_point", 0):
                raise B200CompileError("dequantize with a zero-point after quantized_dot is not supported")
            tensor_scale = float(deq.attrs["scale"])
            absorbed += [deq]
            y = deq.result
        else:
            raise B200CompileError("quantized_dot must be followed by its dequantizing tail")
        bias = None
        add = self.single_user(y, "add")
        if add is not None:
            src = _broadcast_source(self.other(add, y))
            arr = _const_array(src) if src is not None else None
            if arr is not None and arr.size == N:
                bias = arr.reshape(-1).astype(np.float32)
                absorbed.append(add)
                y = add.result
        for o in absorbed:
            self.done.add(id(o))
        act, y, act_ops = self.match_activation(y)
        for o in act_ops:
            self.done.add(id(o))
        if tensor_scale is not None or zp_a or zp_w:
            # Two steps: the int32 contraction (tensor cores; zero-points through the correction terms; ui8 operands
            # shifted by 128) and the tail as its own kernel.  The per-tensor `dequantize` multiplies by a binary64
            # immediate (quant_math.ts:29-34), which the fused kernel's binary32 scale vector cannot reproduce.
            if self.dynamic:
                raise B200CompileError("per_token_dynamic needs the symmetric per-channel form of quantized_dot")
            lhs, _ = self.as_i8(lhs)
            acc = op.result
            self.steps.append(Step("dot", [lhs], acc, {"M": M, "N": N, "K": K, "w": w.astype(np.int8), "w_layout": w_layout,
                                                       "zp_a": zp_a, "zp_w": zp_w}))
            self.steps.append(Step("tail", [acc], y, {"M": M, "N": N, "tensor_scale": tensor_scale, "bias": bias, "act": act,
                                                      "w_scales": None if sv is None else sv.astype(np.float32)}))
            return
        params = {"M": M, "N": N, "K": K, "w": w.astype(np.int8), "w_layout": w_layout, "bias": bias, "act": act,
                  "requant_scale": None, "a_dynamic": False}
        if self.dynamic:
            # recover the weight scales from the baked product (both are still binary64 here), rounded to f32 once
            params["w_scales"] = (sv / lhs_scale).astype(np.float32)
            params["a_dynamic"] = True
        else:
            params["w_scales"] = sv.astype(np.float32)          # fround(aScale * wScale[n]): the f32 constant of the graph
        # a following static quantize of the result fuses into the epilogue
        nq = self.single_user(y, "quantize")
        if nq is not None and not self.dynamic and not nq.attrs.get("zero_point", 0) and nq.attrs.get("target_dtype", "i8") == "i8" \
                and not any(r is y for r in self.f.returns):
            params["requant_scale"] = float(nq.attrs["scale"])
            self.done.add(id(nq))
            y = nq.result
        self.steps.append(Step("linear", [lhs], y, params))

    def materialize(self, v: Value):
        """A constant that a native step reads as a buffer (the kernel of a convolution, the f32 source of its
        `quantize`) becomes a 'const' step: uploaded once when the plan is built."""
        if v.producer is not None and v.producer.name == "constant" and id(v) not in self.consts:
            self.consts.add(id(v))
            self.steps.append(Step("const", [], v, {"data": np.ascontiguousarray(_const_array(v), NP_DTYPE[v.dtype])}))

    def as_i8(self, v: Value):
        """ui8 operands of a contraction: a 'shift' step turns them into int8 codes 128 lower; the caller moves the
        zero-point by the returned amount (u - zp == (u - 128) - (zp - 128))."""
        if v.dtype != "ui8":
            return v, 0
        self.materialize(v)
        shifted = Value(v.shape, "i8")
        self.steps.append(Step("shift", [v], shifted, {"n": int(np.prod(v.shape))}))
        return shifted, 128

    def plan_conv(self, op: Op):
        """quantized_conv (ops/quantization.ts:156-190): both operands are device buffers (the pass quantizes input
        and kernel with `quantize` ops, tests/compiler/passes/quantization/pass.test.js:428-440); the int32 result is
        read by the `dequantize` that follows as a step of its own."""
        x, k = op.operands
        if x.dtype not in ("i8", "ui8") or k.dtype not in ("i8", "ui8"):
            raise B200CompileError("quantized_conv takes i8 / ui8 operands")
        layouts = (op.attrs.get("input_layout", "NCHW"), op.attrs.get("kernel_layout", "OIHW"))
        if layouts not in (("NCHW", "OIHW"), ("NHWC", "OHWI")) or len(x.shape) != 4 or len(k.shape) != 4:
            raise B200CompileError("quantized_conv: two spatial dimensions, layouts NCHW / OIHW or NHWC / OHWI")
        strides = [int(v) for v in op.attrs["strides"]]
        padding = [[int(a), int(b)] for a, b in op.attrs["padding"]]
        dilation = [int(v) for v in (op.attrs.get("dilation") or [1] * len(strides))]
        if layouts[0] == "NCHW":
            (N, C, H, W), (O, _, KH, KW) = x.shape, k.shape
        else:
            (N, H, W, C), (O, KH, KW, _) = x.shape, k.shape
        self.materialize(x)
        self.materialize(k)
        x, sx = self.as_i8(x)
        k, sk = self.as_i8(k)
        self.steps.append(Step("conv", [x, k], op.result, {
            "shape": [N, C, H, W], "kernel_shape": [O, KH, KW], "strides": strides, "padding": padding, "dilation": dilation,
            "groups": int(op.attrs.get("groups") or 1), "zp_in": int(op.attrs.get("input_zero_point", 0) or 0) - sx,
            "zp_ker": int(op.attrs.get("kernel_zero_point", 0) or 0) - sk, "layout": layouts[0]}))

    def plan(self) -> List[Step]:
        for op in self.f.ops:
            if id(op) in self.done:
                continue
            n = op.name
            if n in ("constant", "broadcast_in_dim", "broadcast"):
                continue                       # consumed through their users
            if n == "quantize":
                x = op.operands[0]
                self.materialize(x)
                users = self.f.users(op.result)
                feeds_dot = bool(users) and all(u.name == "quantized_dot" and u.operands[0] is op.result for u in users)
                if self.dynamic and feeds_dot and len(x.shape) >= 2:
                    self.steps.append(Step("quantize_token", [x], op.result, {"K": x.shape[-1], "M": int(np.prod(x.shape[:-1]))}))
                else:
                    self.steps.append(Step("quantize_static", [x], op.result, {
                        "scale": float(op.attrs["scale"]), "zero_point": int(op.attrs.get("zero_point", 0)),
                        "kind": 1 if op.attrs.get("target_dtype", "i8") == "ui8" else 0}))
            elif n == "dequantize":
                self.steps.append(Step("dequantize_static", [op.operands[0]], op.result, {
                    "scale": float(op.attrs["scale"]), "zero_point": int(op.attrs.get("zero_point", 0)),
                    "kind": {"i8": 0, "ui8": 1, "i32": 2}[op.operands[0].dtype]}))
            elif n == "quantized_dot":
                self.plan_dot(op)
            elif n == "quantized_conv":
                self.plan_conv(op)
            elif n == "return":
                continue
            else:
                raise B200CompileError(f"op '{n}' is outside the graph contract of the B200 backend "
                                       "(quantize, dequantize, quantized_dot and its per-channel tail, quantized_conv); "
                                       "compile with quantizableOps = {'dot'} and keep other ops on another target")
        return self.steps


def plan_function(func: GraphFunction, dynamic: bool) -> List[Step]:
    return _Planner(func, dynamic).plan()


# ----------------------------------------------------------------------------- native programs
# A planned function as data: what RuntimeModule.serialize() of the reference keeps per kernel is
# {name, source, target, metadata} (src/runtime/runtime.ts:399-414); for this backend `source` is the JSON text below
# and metadata.kind is 'b200', so a quantized model reloads through RuntimeModule.deserialize() and the 'b200' runtime
# backend without running the quantization pass or the matcher again.  Values are numbered in order of appearance;
# weights, scale vectors and biases travel as base64 of their little-endian bytes.
PROGRAM_VERSION = 1
_ARRAY_PARAMS = {"w": np.int8, "w_scales": np.float32, "bias": np.float32}


def program_of(args: Sequence[Value], returns: Sequence[Value], steps: Sequence[Step]) -> dict:
    import base64
    ids: Dict[int, int] = {}

    def vid(v: Value) -> int:
        if id(v) not in ids:
            ids[id(v)] = len(ids)
        return ids[id(v)]

    out_args = [{"id": vid(v), "shape": list(v.shape), "dtype": v.dtype} for v in args]
    out_steps = []
    for st in steps:
        params = {}
        for k, val in st.params.items():
            if k in ("dW", "dws", "db"):          # device buffers of a live plan are not part of the program
                continue
            if k in _ARRAY_PARAMS or k == "data":
                dt = NP_DTYPE[st.out.dtype] if k == "data" else _ARRAY_PARAMS[k]   # a constant travels in its own dtype
                params[k] = None if val is None else {"shape": list(np.shape(val)),
                                                      "b64": base64.b64encode(np.ascontiguousarray(val, dt).tobytes()).decode("ascii")}
            else:
                params[k] = val
        out_steps.append({"kind": st.kind, "ins": [vid(v) for v in st.ins],
                          "out": {"id": vid(st.out), "shape": list(st.out.shape), "dtype": st.out.dtype}, "params": params})
    return {"version": PROGRAM_VERSION, "args": out_args, "steps": out_steps, "returns": [vid(v) for v in returns]}


def steps_from_program(program: dict):
    """(args, returns, steps) rebuilt from :func:`program_of` output (after a trip through JSON)."""
    import base64
    if program.get("version") != PROGRAM_VERSION:
        raise B200CompileError(f"native program version {program.get('version')} is not understood (this build reads {PROGRAM_VERSION})")
    vals: Dict[int, Value] = {}
    args = []
    for a in program["args"]:
        vals[a["id"]] = Value(tuple(a["shape"]), a["dtype"], None, f"arg{len(args)}")
        args.append(vals[a["id"]])
    steps = []
    for st in program["steps"]:
        if st["kind"] not in ("quantize_static", "quantize_token", "dequantize_static", "linear", "dot", "tail", "conv", "const", "shift"):
            raise B200CompileError(f"native program: unknown step '{st['kind']}'")
        o = st["out"]
        vals[o["id"]] = Value(tuple(o["shape"]), o["dtype"])
        params = {}
        for k, val in st["params"].items():
            if (k in _ARRAY_PARAMS or k == "data") and val is not None:
                dt = NP_DTYPE[o["dtype"]] if k == "data" else _ARRAY_PARAMS[k]
                params[k] = np.frombuffer(base64.b64decode(val["b64"]), dt).reshape(val["shape"]).copy()
            else:
                params[k] = val
        try:
            ins = [vals[i] for i in st["ins"]]
        except KeyError as exc:
            raise B200CompileError(f"native program: step reads value {exc} before it is produced") from None
        steps.append(Step(st["kind"], ins, vals[o["id"]], params))
    try:
        returns = [vals[i] for i in program["returns"]]
    except KeyError as exc:
        raise B200CompileError(f"native program: returned value {exc} is never produced") from None
    return args, returns, steps


# ----------------------------------------------------------------------------- execution
class _Signature:
    """What a plan needs of a function once it is planned: its arguments and returned values."""

    def __init__(self, args, returns):
        self.args, self.returns = list(args), list(returns)


class _FunctionPlan:
    def __init__(self, ctx: Context, func, dynamic: bool = False, steps: Optional[List[Step]] = None):
        self.func = func
        self.steps = plan_function(func, dynamic) if steps is None else steps
        self.inputs = len(func.args)
        self.outputs = len(func.returns)
        self.ctx = ctx
        self.buf: Dict[int, Any] = {}           # id(Value) -> DeviceBuffer
        self.scales: Dict[int, Any] = {}        # id(Value of per-token codes) -> DeviceBuffer of scales
        for v in func.args:
            self._alloc(v)
        for st in self.steps:
            self._alloc(st.out)
            if st.kind == "quantize_token":
                self.scales[id(st.out)] = ctx.empty((st.params["M"],), np.float32)
            if st.kind == "const":
                self.buf[id(st.out)].upload(np.ascontiguousarray(st.params["data"], NP_DTYPE[st.out.dtype]).reshape(st.out.shape if st.out.shape else (1,)))
            if st.kind in ("linear", "dot"):
                p = st.params
                w = p["w"]
                if p["w_layout"] == W_KN:       # re-lay [K,N] constants as [N,K] once, on the device
                    src = ctx.to_device(w)
                    dst = ctx.empty((p["N"], p["K"]), np.int8)
                    ctx.transpose_i8(src, p["K"], p["N"], dst)
                    ctx.sync()
                    src.free()
                    p["dW"] = dst
                else:
                    p["dW"] = ctx.to_device(w)
                if st.kind == "linear":
                    p["dws"] = ctx.to_device(p["w_scales"])
                    p["db"] = ctx.to_device(p["bias"]) if p["bias"] is not None else None
            if st.kind == "tail":
                p = st.params
                p["dws"] = ctx.to_device(p["w_scales"]) if p["w_scales"] is not None else None
                p["db"] = ctx.to_device(p["bias"]) if p["bias"] is not None else None
        missing = [r for r in func.returns if id(r) not in self.buf]
        if missing:
            raise B200CompileError("a returned value is not produced by any native step")

    @classmethod
    def from_program(cls, ctx: Context, program: dict) -> "_FunctionPlan":
        args, returns, steps = steps_from_program(program)
        return cls(ctx, _Signature(args, returns), steps=steps)

    def program(self) -> dict:
        return program_of(self.func.args, self.func.returns, self.steps)

    def _alloc(self, v: Value):
        if id(v) not in self.buf:
            self.buf[id(v)] = self.ctx.empty(v.shape if v.shape else (1,), NP_DTYPE[v.dtype])

    def describe(self) -> str:
        lines = []
        for st in self.steps:
            p = {k: v for k, v in st.params.items() if k in ("M", "N", "K", "act", "scale", "zero_point", "requant_scale", "a_dynamic")}
            lines.append(f"{st.kind} {p}")
        return "\n".join(lines)

    def execute(self, arrays: Sequence[np.ndarray]):
        ctx = self.ctx
        for v, a in zip(self.func.args, arrays[: self.inputs]):
            self.buf[id(v)].upload(np.ascontiguousarray(a, NP_DTYPE[v.dtype]).reshape(v.shape))
        for st in self.steps:
            if st.kind == "const":              # uploaded when the plan was built
                continue
            x = self.buf[id(st.ins[0])]
            out = self.buf[id(st.out)]
            p = st.params
            if st.kind == "shift":
                ctx.shift_u8_to_i8(x, p["n"], out)
            elif st.kind == "conv":
                ctx.quantized_conv2d(x, self.buf[id(st.ins[1])], p["shape"], p["kernel_shape"], out, p["strides"], p["padding"],
                                     p["dilation"], p["groups"], p["zp_in"], p["zp_ker"], p["layout"])
            elif st.kind == "dot":
                ctx.int8_gemm_i32(x, p["dW"], p["M"], p["N"], p["K"], out, p["zp_a"], p["zp_w"])
            elif st.kind == "tail":
                if p["dws"] is not None:
                    ctx.epilogue(x, p["M"], p["N"], None, p["dws"], p["db"], p["act"], out)
                else:
                    ctx.epilogue_tensor_scale(x, p["M"], p["N"], p["tensor_scale"], p["db"], p["act"], out)
            elif st.kind == "quantize_static":
                ctx.quantize_static(x, int(np.prod(st.ins[0].shape)), p["scale"], p["zero_point"], p["kind"], out)
            elif st.kind == "quantize_token":
                ctx.quantize_per_token(x, p["M"], p["K"], out, self.scales[id(st.out)])
            elif st.kind == "dequantize_static":
                ctx.dequantize_static(x, p["kind"], int(np.prod(st.ins[0].shape)), p["scale"], p["zero_point"], out)
            elif st.kind == "linear":
                a_scales = self.scales.get(id(st.ins[0])) if p["a_dynamic"] else None
                if p["a_dynamic"] and a_scales is None:
                    raise B200CompileError("dynamic activation scales are missing for a quantized_dot operand")
                if p["requant_scale"] is not None:
                    ctx.int8_linear_requant_static(x, a_scales, p["dW"], p["dws"], p["db"], p["act"], p["M"], p["N"], p["K"],
                                                   p["requant_scale"], out)
                else:
                    ctx.int8_linear(x, a_scales, p["dW"], p["dws"], p["db"], p["act"], p["M"], p["N"], p["K"], out)
        ctx.sync()
        ctx.check_status()
        for v, a in zip(self.func.returns, arrays[self.inputs:]):
            res = self.buf[id(v)].download()
            np.copyto(a.reshape(res.shape), res)


def _as_array(arg) -> np.ndarray:
    """Both argument forms of the reference (src/runtime/runtime.ts:242-250): a typed array or {data, shape, dtype}."""
    if isinstance(arg, np.ndarray):
        return arg
    if isinstance(arg, dict) and "data" in arg:
        return np.asarray(arg["data"]).reshape(arg.get("shape", np.asarray(arg["data"]).shape))
    raise TypeError("arguments must be numpy arrays or {data, shape, dtype} tensors")


class B200RuntimeModule:
    """RuntimeModuleLike over libb200q.so: one native plan per function of the module."""

    def __init__(self, module: Dict[str, GraphFunction], options: Optional[dict] = None, _programs: Optional[dict] = None):
        options = options or {}
        self.name = options.get("name", "module")
        self.ctx = Context(int(options.get("device", 0) or 0))      # raises without a GPU: no fallback
        if _programs is not None:
            self.plans = {name: _FunctionPlan.from_program(self.ctx, prog) for name, prog in _programs.items()}
            return
        dynamic = options.get("activationQuant", "static") == "per_token_dynamic"
        self.plans = {name: _FunctionPlan(self.ctx, f, dynamic) for name, f in module.items()}

    def serialize(self) -> dict:
        """``SerializedRuntimeModule`` of the reference (src/runtime/runtime.ts:399-406): one entry per function whose
        ``source`` is the native program as JSON text."""
        import json
        return {"name": self.name, "kernels": [
            {"name": name, "source": json.dumps(p.program()), "target": "b200_int8",
             "metadata": {"kind": "b200", "inputs": p.inputs, "outputs": p.outputs, "steps": len(p.steps)}}
            for name, p in self.plans.items()]}

    @classmethod
    def deserialize(cls, data: dict, options: Optional[dict] = None) -> "B200RuntimeModule":
        """The counterpart of ``RuntimeModule.deserialize`` (runtime.ts:408-414): rebuilds the plans from the stored
        programs - weights and scales are uploaded as they are, nothing is quantized or matched again."""
        import json
        programs = {}
        for k in data["kernels"]:
            if k.get("metadata", {}).get("kind") != "b200":
                raise B200CompileError(f"kernel '{k.get('name')}' is of kind {k.get('metadata', {}).get('kind')!r}, not 'b200'")
            programs[k["name"]] = json.loads(k["source"])
        return cls({}, {**(options or {}), "name": data.get("name", "module")}, _programs=programs)

    def run(self, funcName: str, *args):
        plan = self.plans.get(funcName)
        if plan is None:
            raise KeyError(f"b200: no function named {funcName}")
        if len(args) != plan.inputs + plan.outputs:
            raise ValueError(f"b200: {funcName} takes {plan.inputs} tensors and returns {plan.outputs}, "
                             f"but the call passes {len(args)} buffers")
        plan.execute([_as_array(a) for a in args])

    def runAsync(self, funcName: str, *args):
        return self.run(funcName, *args)

    def isAsync(self, funcName: str = "") -> bool:
        return False

    def getKernelSource(self, funcName: str) -> Optional[str]:
        p = self.plans.get(funcName)
        return p.describe() if p else None

    def getKernelMetadata(self, funcName: str) -> Optional[dict]:
        p = self.plans.get(funcName)
        return {"kind": "b200", "inputs": p.inputs, "outputs": p.outputs, "steps": len(p.steps)} if p else None

    def listKernels(self) -> List[str]:
        return list(self.plans)

    def release(self):
        if self.ctx is not None:
            self.ctx.close()
            self.ctx = None
