// planGraph: matches the post-pass graph against the backend's graph contract and turns every function
// into a list of native steps.  A transliteration of plan_function / _FunctionPlan in mlfw_b200/backend.py,
// which is the tested form of the same rules (no JavaScript engine exists in the build image).
//
// Contract (what QuantizationPass emits with fusion disabled on the target,
// src/compiler/passes/quantization/quantization_pass.ts:286-459):
//   quantize · quantized_dot(constant i8 rhs) · convert · mul(broadcast_in_dim(constant f32[N]))
//   [· add(broadcast(bias))] [· maximum(·,0) | x·sigmoid(1.702x) | x·sigmoid(x)] [· quantize]   -> one 'linear' step
//   quantize(x) · quantize(kernel) · quantized_conv  -> 'conv' (int32; the `dequantize` after it is a step of its own)
//   quantized_dot{zero-points} (asymmetric operands)  -> 'dot' (int32 on the tensor cores plus the zero-point terms)
//   quantized_dot · dequantize{scale} [· add · activation]   -> 'dot' + 'tail' (the scale is a binary64 immediate: quant_math.ts:29-34)
//   standalone quantize / dequantize                                                                 -> static steps
// Anything else throws: the backend has no fallback.
import { check } from './binding.js';

import type { B200QBinding } from './binding.js';
import type { GraphModule } from '../../compiler/ir/graph/module.js';
import type { GraphFunction } from '../../compiler/ir/graph/function.js';
import type { Operation } from '../../compiler/ir/graph/operation.js';
import type { Value } from '../../compiler/ir/graph/value.js';
import type { B200Options } from './target.js';

const ACT = { none: 0, relu: 1, gelu_sigmoid: 2, gelu_tanh: 3, silu: 4 } as const;
type Act = keyof typeof ACT;
type Step =
  | { kind: 'quantize_static'; in: Value; out: Value; scale: number; zeroPoint: number; dst: number }
  | { kind: 'quantize_token'; in: Value; out: Value; M: number; K: number }
  | { kind: 'dequantize_static'; in: Value; out: Value; scale: number; zeroPoint: number; src: number }
  | { kind: 'linear'; in: Value; out: Value; M: number; N: number; K: number; act: Act; dynamic: boolean;
      w: Int8Array; wIsKN: boolean; wScales: Float32Array; bias: Float32Array | null; requantScale: number | null;
      dW?: unknown; dWs?: unknown; dBias?: unknown }
  // quantized_dot with zero-points (asymmetric operands): the int32 contraction alone; the `dequantize` after it is a static step
  | { kind: 'dot'; in: Value; out: Value; M: number; N: number; K: number; w: Int8Array; wIsKN: boolean; zpA: number; zpW: number; dW?: unknown }
  // the tail of a 'dot' as its own kernel: a per-channel binary32 scale vector, or the one binary64 scale of a per-tensor `dequantize`
  | { kind: 'tail'; in: Value; out: Value; M: number; N: number; tensorScale: number | null; wScales: Float32Array | null; bias: Float32Array | null; act: Act;
      dWs?: unknown; dBias?: unknown }
  // a ui8 operand of a contraction as int8 codes 128 lower (the zero-point moves along: u - zp == (u - 128) - (zp - 128))
  | { kind: 'shift'; in: Value; out: Value; n: number }
  // a constant that a native step reads as a buffer (a convolution's kernel, the f32 source of its `quantize`): uploaded once
  | { kind: 'const'; out: Value; data: ArrayBufferView }
  // quantized_conv (ops/quantization.ts:156-190): both operands are device buffers, the int32 result feeds a `dequantize`
  | { kind: 'conv'; in: Value; ker: Value; out: Value; shape: number[]; kernelShape: number[]; strides: number[]; padding: number[][];
      dilation: number[]; groups: number; zpIn: number; zpKer: number; layout: 'NCHW' | 'NHWC' };
const TYPED = { f32: Float32Array, i32: Int32Array, i8: Int8Array, ui8: Uint8Array } as const;

const shapeOf = (v: Value): number[] => (v.type as { shape: number[] }).shape;
const dtypeOf = (v: Value): string => (v.type as { dtype: string }).dtype;
const numel = (s: readonly number[]) => s.reduce((a, b) => a * b, 1);

function users(f: GraphFunction, v: Value, done: Set<Operation>): Operation[] {
  const out: Operation[] = [];
  for (const op of f.ops()) if (!done.has(op)) for (let i = 0; i < op.numOperands; i++) if (op.getOperand(i) === v) { out.push(op); break; }
  return out;
}
function broadcastSource(v: Value): Value | null {
  const d = v.definingOp;
  if (!d) return null;
  if (d.opName === 'broadcast_in_dim' || d.opName === 'broadcast') return d.getOperand(0);
  return d.opName === 'constant' ? v : null;
}
function constArray(v: Value | null): number[] | null {
  const d = v?.definingOp;
  if (!d || d.opName !== 'constant') return null;
  const val = d.getAttr<number | number[]>('value');
  return typeof val === 'number' ? [val] : [...(val as number[])];
}
const scalarConst = (v: Value): number | null => { const a = constArray(broadcastSource(v)); return a && a.length === 1 ? a[0] : null; };
const other = (op: Operation, v: Value): Value => (op.getOperand(0) === v ? op.getOperand(1) : op.getOperand(0));

function matchSigmoid(f: GraphFunction, z: Value, done: Set<Operation>): { res: Value; ops: Operation[] } | null {
  const neg = users(f, z, done).find((u) => u.opName === 'neg'); if (!neg) return null;
  const exp = users(f, neg.getResult(0), done); if (exp.length !== 1 || exp[0].opName !== 'exp') return null;
  const add = users(f, exp[0].getResult(0), done); if (add.length !== 1 || add[0].opName !== 'add' || scalarConst(other(add[0], exp[0].getResult(0))) !== 1) return null;
  const div = users(f, add[0].getResult(0), done);
  if (div.length !== 1 || div[0].opName !== 'div' || div[0].getOperand(1) !== add[0].getResult(0) || scalarConst(div[0].getOperand(0)) !== 1) return null;
  return { res: div[0].getResult(0), ops: [neg, exp[0], add[0], div[0]] };
}

function matchActivation(f: GraphFunction, y: Value, done: Set<Operation>): { act: Act; res: Value; ops: Operation[] } {
  const us = users(f, y, done);
  if (us.length === 1 && us[0].opName === 'maximum' && scalarConst(other(us[0], y)) === 0) return { act: 'relu', res: us[0].getResult(0), ops: [us[0]] };
  const silu = matchSigmoid(f, y, done);
  if (silu) {
    const mul = users(f, silu.res, done).find((u) => u.opName === 'mul' && (u.getOperand(0) === y || u.getOperand(1) === y));
    if (mul) return { act: 'silu', res: mul.getResult(0), ops: [...silu.ops, mul] };
  }
  for (const u of us) {
    if (u.opName !== 'mul') continue;
    const c = scalarConst(other(u, y));
    if (c === null || Math.abs(c - 1.702) > 1e-12) continue;
    const sig = matchSigmoid(f, u.getResult(0), done);
    const mul = sig && users(f, sig.res, done).find((m) => m.opName === 'mul' && (m.getOperand(0) === y || m.getOperand(1) === y));
    if (sig && mul) return { act: 'gelu_sigmoid', res: mul.getResult(0), ops: [u, ...sig.ops, mul] };
  }
  return { act: 'none', res: y, ops: [] };
}

function planFunction(f: GraphFunction, dynamic: boolean): Step[] {
  const steps: Step[] = [];
  const done = new Set<Operation>();
  const returns = new Set<Value>(f.returnValues());
  const consts = new Set<Value>();
  const materialize = (v: Value) => {
    const a = constArray(v);
    if (!a || consts.has(v)) return;
    consts.add(v);
    steps.push({ kind: 'const', out: v, data: TYPED[dtypeOf(v) as keyof typeof TYPED].from(a) });
  };
  const shifted = new Map<Value, Value>();
  const asI8 = (v: Value): [Value, number] => {         // shifted values are keyed by a stand-in object for the new buffer
    if (dtypeOf(v) !== 'ui8') return [v, 0];
    materialize(v);
    if (!shifted.has(v)) {
      const nv = { type: { shape: shapeOf(v), dtype: 'i8' } } as unknown as Value;
      shifted.set(v, nv);
      steps.push({ kind: 'shift', in: v, out: nv, n: numel(shapeOf(v)) });
    }
    return [shifted.get(v)!, 128];
  };
  for (const op of f.ops()) {
    if (done.has(op)) continue;
    const n = op.opName;
    if (n === 'constant' || n === 'broadcast_in_dim' || n === 'broadcast' || n === 'return') continue;
    if (n === 'quantize') {
      const x = op.getOperand(0), us = users(f, op.getResult(0), done);
      const feedsDot = us.length > 0 && us.every((u) => u.opName === 'quantized_dot' && u.getOperand(0) === op.getResult(0));
      const s = shapeOf(x);
      materialize(x);
      if (dynamic && feedsDot && s.length >= 2) steps.push({ kind: 'quantize_token', in: x, out: op.getResult(0), M: numel(s.slice(0, -1)), K: s[s.length - 1] });
      else steps.push({ kind: 'quantize_static', in: x, out: op.getResult(0), scale: op.getAttr<number>('scale')!, zeroPoint: op.getAttr<number>('zero_point') || 0,
                        dst: op.getAttr<string>('target_dtype') === 'ui8' ? 1 : 0 });
    } else if (n === 'dequantize') {
      steps.push({ kind: 'dequantize_static', in: op.getOperand(0), out: op.getResult(0), scale: op.getAttr<number>('scale')!, zeroPoint: op.getAttr<number>('zero_point') || 0,
                   src: { i8: 0, ui8: 1, i32: 2 }[dtypeOf(op.getOperand(0)) as 'i8' | 'ui8' | 'i32'] });
    } else if (n === 'quantized_dot') {
      const lhs = op.getOperand(0), rhs = op.getOperand(1);
      const w = constArray(rhs), rs = shapeOf(rhs), ls = shapeOf(lhs);
      if (!w || (dtypeOf(rhs) !== 'i8' && dtypeOf(rhs) !== 'ui8') || rs.length !== 2) throw new Error('b200: quantized_dot needs a constant rank-2 int8 rhs');
      const rc = op.getAttr<number[]>('rhs_contracting') || [0];
      const K = rs[rc[0]], N = rs[1 - rc[0]], M = numel(ls.slice(0, -1));
      let zpA = op.getAttr<number>('lhs_zero_point') || 0, zpW = op.getAttr<number>('rhs_zero_point') || 0;
      const wI8 = dtypeOf(rhs) === 'ui8' ? w.map((v) => v - 128) : w;       // constant ui8 codes: moved by 128 here, on the host
      if (dtypeOf(rhs) === 'ui8') zpW -= 128;
      if (dtypeOf(lhs) === 'ui8') zpA -= 128;
      const lhsScale = op.getAttr<number>('lhs_scale') || 1;
      let y = op.getResult(0), sv: number[] | null = null, tensorScale: number | null = null;
      done.add(op);
      const next = users(f, y, done);
      if (next.length === 1 && next[0].opName === 'convert') {
        const mul = users(f, next[0].getResult(0), done);
        const arr = mul.length === 1 && mul[0].opName === 'mul' ? constArray(broadcastSource(other(mul[0], next[0].getResult(0)))) : null;
        if (!arr || arr.length !== N) throw new Error('b200: quantized_dot -> convert must be followed by mul with a per-channel scale vector');
        sv = arr; done.add(next[0]); done.add(mul[0]); y = mul[0].getResult(0);
      } else if (next.length === 1 && next[0].opName === 'dequantize' && !next[0].getAttr<number>('zero_point')) {
        tensorScale = next[0].getAttr<number>('scale')!; done.add(next[0]); y = next[0].getResult(0);
      } else throw new Error('b200: quantized_dot must be followed by its dequantizing tail');
      let bias: Float32Array | null = null;
      const add = users(f, y, done);
      if (add.length === 1 && add[0].opName === 'add') {
        const arr = constArray(broadcastSource(other(add[0], y)));
        if (arr && arr.length === N) { bias = Float32Array.from(arr); done.add(add[0]); y = add[0].getResult(0); }
      }
      const a = matchActivation(f, y, done);
      a.ops.forEach((o) => done.add(o)); y = a.res;
      if (tensorScale !== null || zpA || zpW) {
        // two steps: the int32 contraction (zero-points through correction terms, ui8 operands shifted) and the tail as
        // its own kernel; the per-tensor `dequantize` multiplies by a binary64 immediate (quant_math.ts:29-34)
        if (dynamic) throw new Error('b200: per_token_dynamic needs the symmetric per-channel form of quantized_dot');
        const [lhsI8] = asI8(lhs);
        const acc = op.getResult(0);
        steps.push({ kind: 'dot', in: lhsI8, out: acc, M, N, K, w: Int8Array.from(wI8), wIsKN: rc[0] === 0, zpA, zpW });
        steps.push({ kind: 'tail', in: acc, out: y, M, N, tensorScale, wScales: sv ? Float32Array.from(sv) : null, bias, act: a.act });
        continue;
      }
      // dynamic per-token: recover wScale[n] = scaleVec[n] / lhs_scale (both binary64 here), rounded to f32 once
      const wScales = Float32Array.from(dynamic ? sv!.map((s) => s / lhsScale) : sv!);
      let requantScale: number | null = null;
      const nq = users(f, y, done);
      if (!dynamic && nq.length === 1 && nq[0].opName === 'quantize' && !nq[0].getAttr<number>('zero_point') && !returns.has(y)) {
        requantScale = nq[0].getAttr<number>('scale')!; done.add(nq[0]); y = nq[0].getResult(0);
      }
      steps.push({ kind: 'linear', in: lhs, out: y, M, N, K, act: a.act, dynamic, w: Int8Array.from(w), wIsKN: rc[0] === 0, wScales, bias, requantScale });
    } else if (n === 'quantized_conv') {
      const x = op.getOperand(0), k = op.getOperand(1), xs = shapeOf(x), ks = shapeOf(k);
      if (!['i8', 'ui8'].includes(dtypeOf(x)) || !['i8', 'ui8'].includes(dtypeOf(k))) throw new Error('b200: quantized_conv takes i8 / ui8 operands');
      const il = op.getAttr<string>('input_layout') || 'NCHW', kl = op.getAttr<string>('kernel_layout') || 'OIHW';
      if (!((il === 'NCHW' && kl === 'OIHW') || (il === 'NHWC' && kl === 'OHWI')) || xs.length !== 4 || ks.length !== 4)
        throw new Error('b200: quantized_conv: two spatial dimensions, layouts NCHW / OIHW or NHWC / OHWI');
      const strides = op.getAttr<number[]>('strides')!, padding = op.getAttr<number[][]>('padding')!;
      const first = il === 'NCHW';
      materialize(x); materialize(k);
      const [xI8, sx] = asI8(x), [kI8, sk] = asI8(k);
      steps.push({ kind: 'conv', in: xI8, ker: kI8, out: op.getResult(0),
                   shape: first ? xs : [xs[0], xs[3], xs[1], xs[2]], kernelShape: first ? [ks[0], ks[2], ks[3]] : [ks[0], ks[1], ks[2]],
                   strides, padding, dilation: op.getAttr<number[]>('dilation') || strides.map(() => 1), groups: op.getAttr<number>('groups') || 1,
                   zpIn: (op.getAttr<number>('input_zero_point') || 0) - sx, zpKer: (op.getAttr<number>('kernel_zero_point') || 0) - sk, layout: il as 'NCHW' | 'NHWC' });
    } else {
      throw new Error(`b200: op '${n}' is outside the graph contract (quantize, dequantize, quantized_dot and its tail, quantized_conv)`);
    }
  }
  return steps;
}

type ConvParams = { shape: number[]; kernelShape: number[]; strides: number[]; padding: number[][]; dilation: number[]; groups: number;
                    zpIn: number; zpKer: number; layout: string };
function runConv(b: B200QBinding, c: unknown, x: unknown, k: unknown, y: unknown, q: ConvParams): void {
  const [N, C, H, W] = q.shape, [O, KH, KW] = q.kernelShape;
  check(b, b.quantizedConv2d(c, x, k, N, C, H, W, O, KH, KW, q.strides[0], q.strides[1], q.padding[0][0], q.padding[0][1], q.padding[1][0],
                             q.padding[1][1], q.dilation[0], q.dilation[1], q.groups, q.zpIn, q.zpKer, q.layout === 'NHWC' ? 1 : 0, y), 'b200q_quantized_conv2d');
}

export type FunctionPlan = { inputs: number; outputs: number; steps: Step[]; describe(): string; execute(b: B200QBinding, ctx: unknown, args: ArrayBufferView[]): void };

export function planGraph(module: GraphModule, options: B200Options, b: B200QBinding, ctx: unknown): Map<string, FunctionPlan> {
  const dynamic = options.activationQuant === 'per_token_dynamic';
  const plans = new Map<string, FunctionPlan>();
  const alloc = (bytes: number): unknown => { const out: [unknown] = [null]; check(b, b.alloc(ctx, bytes, out), 'b200q_alloc'); return out[0]; };
  const upload = (a: ArrayBufferView): unknown => { const d = alloc(a.byteLength); check(b, b.upload(ctx, d, a, a.byteLength), 'b200q_upload'); return d; };
  const bytesOf = (v: Value) => numel(shapeOf(v)) * ({ f32: 4, i32: 4, i8: 1, ui8: 1 } as Record<string, number>)[dtypeOf(v)];
  for (const f of module.functions()) {
    const steps = planFunction(f, dynamic);
    const buf = new Map<Value, unknown>(), tokScales = new Map<Value, unknown>();
    for (const v of f.args) buf.set(v, alloc(bytesOf(v)));
    for (const st of steps) {
      if (st.kind === 'const') { buf.set(st.out, upload(st.data)); continue; }
      buf.set(st.out, alloc(bytesOf(st.out)));
      if (st.kind === 'quantize_token') tokScales.set(st.out, alloc(st.M * 4));
      if (st.kind === 'linear' || st.kind === 'dot') { // weights cross the boundary once, as buffers
        const raw = upload(st.w);
        if (st.wIsKN) { st.dW = alloc(st.w.byteLength); check(b, b.transposeI8(ctx, raw, st.K, st.N, st.dW), 'b200q_transpose_i8'); check(b, b.sync(ctx), 'b200q_sync'); check(b, b.free(ctx, raw), 'b200q_free'); }
        else st.dW = raw;
      }
      if (st.kind === 'linear') {
        st.dWs = upload(st.wScales);
        st.dBias = st.bias ? upload(st.bias) : null;
      }
      if (st.kind === 'tail') {
        st.dWs = st.wScales ? upload(st.wScales) : null;
        st.dBias = st.bias ? upload(st.bias) : null;
      }
    }
    const rets = f.returnValues();
    plans.set(f.name, {
      inputs: f.args.length, outputs: rets.length, steps,
      describe: () => steps.map((s) => s.kind).join('\n'),
      execute(bind, c, args) {
        f.args.forEach((v, i) => check(bind, bind.upload(c, buf.get(v), args[i], args[i].byteLength), 'b200q_upload'));
        for (const st of steps) {
          if (st.kind === 'const') continue;              // uploaded when the plan was built
          const x = buf.get(st.in), y = buf.get(st.out);
          if (st.kind === 'conv') runConv(bind, c, x, buf.get(st.ker), y, st);
          else if (st.kind === 'shift') check(bind, bind.shiftU8ToI8(c, x, st.n, y), 'b200q_shift_u8_to_i8');
          else if (st.kind === 'dot') check(bind, bind.int8GemmI32(c, x, st.dW, st.M, st.N, st.K, st.zpA, st.zpW, y), 'b200q_int8_gemm_i32');
          else if (st.kind === 'tail') {
            if (st.dWs) check(bind, bind.epilogue(c, x, st.M, st.N, null, st.dWs, st.dBias, ACT[st.act], y), 'b200q_epilogue');
            else check(bind, bind.epilogueTensorScale(c, x, st.M, st.N, st.tensorScale!, st.dBias, ACT[st.act], y), 'b200q_epilogue_tensor_scale');
          } else if (st.kind === 'quantize_static') check(bind, bind.quantizeStatic(c, x, numel(shapeOf(st.in)), st.scale, st.zeroPoint, st.dst, y), 'b200q_quantize_static');
          else if (st.kind === 'quantize_token') check(bind, bind.quantizePerToken(c, x, st.M, st.K, y, tokScales.get(st.out), -127, 127), 'b200q_quantize_per_token');
          else if (st.kind === 'dequantize_static') check(bind, bind.dequantizeStatic(c, x, st.src, numel(shapeOf(st.in)), st.scale, st.zeroPoint, y), 'b200q_dequantize_static');
          else if (st.requantScale !== null) check(bind, bind.int8LinearRequantStatic(c, x, null, st.dW, st.dWs, st.dBias, ACT[st.act], st.M, st.N, st.K, st.requantScale, y), 'b200q_int8_linear_requant_static');
          else check(bind, bind.int8Linear(c, x, st.dynamic ? tokScales.get(st.in) : null, st.dW, st.dWs, st.dBias, ACT[st.act], st.M, st.N, st.K, y), 'b200q_int8_linear');
        }
        check(bind, bind.sync(c), 'b200q_sync');
        rets.forEach((v, i) => { const a = args[f.args.length + i]; check(bind, bind.download(c, a, buf.get(v), a.byteLength), 'b200q_download'); });
      },
    });
  }
  return plans;
}

// ---------------------------------------------------------------------------------------------- native programs
// A planned function as data: what RuntimeModule.serialize() keeps per kernel is {name, source, target, metadata}
// (src/runtime/runtime.ts:399-414); for this backend `source` is JSON.stringify(programOf(...)) and metadata.kind is
// 'b200', so a quantized model reloads through RuntimeModule.deserialize() and the 'b200' runtime backend
// (register.ts) without running the quantization pass or the matcher again.  Same format as program_of /
// steps_from_program in mlfw_b200/backend.py: values numbered in order of appearance, arrays as base64.
export const PROGRAM_VERSION = 1;
type ValueRec = { id: number; shape: number[]; dtype: string };
export type NativeProgram = { version: number; args: ValueRec[]; returns: number[];
                              steps: { kind: Step['kind']; ins: number[]; out: ValueRec; params: Record<string, unknown> }[] };

const b64 = (a: ArrayBufferView) => ({ shape: [a.byteLength / (a as unknown as { BYTES_PER_ELEMENT: number }).BYTES_PER_ELEMENT],
                                       b64: Buffer.from(a.buffer, a.byteOffset, a.byteLength).toString('base64') });
const unb64 = <T>(rec: { b64: string } | null, make: (b: ArrayBuffer) => T): T | null => {
  if (!rec) return null;
  const buf = Buffer.from(rec.b64, 'base64');
  return make(buf.buffer.slice(buf.byteOffset, buf.byteOffset + buf.byteLength));
};

export function programOf(f: GraphFunction, steps: Step[]): NativeProgram {
  const ids = new Map<Value, number>();
  const vid = (v: Value) => { if (!ids.has(v)) ids.set(v, ids.size); return ids.get(v)!; };
  const rec = (v: Value): ValueRec => ({ id: vid(v), shape: shapeOf(v), dtype: dtypeOf(v) });
  const args = f.args.map(rec);
  const out = steps.map((st) => {
    const params: Record<string, unknown> = {};
    if (st.kind === 'linear') Object.assign(params, { M: st.M, N: st.N, K: st.K, act: st.act, a_dynamic: st.dynamic, requant_scale: st.requantScale,
      w_layout: st.wIsKN ? 1 : 0, w: { ...b64(st.w), shape: st.wIsKN ? [st.K, st.N] : [st.N, st.K] }, w_scales: b64(st.wScales), bias: st.bias ? b64(st.bias) : null });
    else if (st.kind === 'quantize_token') Object.assign(params, { M: st.M, K: st.K });
    else if (st.kind === 'quantize_static') Object.assign(params, { scale: st.scale, zero_point: st.zeroPoint, kind: st.dst });
    else if (st.kind === 'dot') Object.assign(params, { M: st.M, N: st.N, K: st.K, zp_a: st.zpA, zp_w: st.zpW, w_layout: st.wIsKN ? 1 : 0,
      w: { ...b64(st.w), shape: st.wIsKN ? [st.K, st.N] : [st.N, st.K] } });
    else if (st.kind === 'const') return { kind: st.kind, ins: [], out: rec(st.out), params: { data: { ...b64(st.data), shape: shapeOf(st.out) } } };
    else if (st.kind === 'shift') Object.assign(params, { n: st.n });
    else if (st.kind === 'tail') Object.assign(params, { M: st.M, N: st.N, tensor_scale: st.tensorScale, act: st.act,
      w_scales: st.wScales ? b64(st.wScales) : null, bias: st.bias ? b64(st.bias) : null });
    else if (st.kind === 'conv') {
      Object.assign(params, { shape: st.shape, kernel_shape: st.kernelShape, strides: st.strides, padding: st.padding, dilation: st.dilation,
                              groups: st.groups, zp_in: st.zpIn, zp_ker: st.zpKer, layout: st.layout });
      return { kind: st.kind, ins: [vid(st.in), vid(st.ker)], out: rec(st.out), params };
    } else Object.assign(params, { scale: st.scale, zero_point: st.zeroPoint, kind: st.src });
    return { kind: st.kind, ins: [vid(st.in)], out: rec(st.out), params };
  });
  return { version: PROGRAM_VERSION, args, steps: out, returns: f.returnValues().map(vid) };
}

/** A FunctionPlan straight from a stored program: weights, scale vectors and biases are uploaded as they are. */
export function planFromProgram(p: NativeProgram, b: B200QBinding, ctx: unknown): FunctionPlan {
  if (p.version !== PROGRAM_VERSION) throw new Error(`b200: native program version ${p.version} is not understood`);
  const alloc = (bytes: number): unknown => { const out: [unknown] = [null]; check(b, b.alloc(ctx, bytes, out), 'b200q_alloc'); return out[0]; };
  const upload = (a: ArrayBufferView): unknown => { const d = alloc(a.byteLength); check(b, b.upload(ctx, d, a, a.byteLength), 'b200q_upload'); return d; };
  const size = (v: ValueRec) => numel(v.shape) * ({ f32: 4, i32: 4, i8: 1, ui8: 1 } as Record<string, number>)[v.dtype];
  const buf = new Map<number, unknown>(), scales = new Map<number, unknown>(), elems = new Map<number, number>();
  for (const a of p.args) { buf.set(a.id, alloc(size(a))); elems.set(a.id, numel(a.shape)); }
  const dev = p.steps.map((st) => {
    const q = st.params as Record<string, any>;
    elems.set(st.out.id, numel(st.out.shape));
    if (st.kind === 'const') { buf.set(st.out.id, upload(unb64(q.data, (x) => new Uint8Array(x))!)); return null; }
    buf.set(st.out.id, alloc(size(st.out)));
    if (st.kind === 'quantize_token') scales.set(st.out.id, alloc(q.M * 4));
    if (st.kind === 'tail') {
      const ws = unb64(q.w_scales, (x) => new Float32Array(x)), tb = unb64(q.bias, (x) => new Float32Array(x));
      return { dW: null, dWs: ws ? upload(ws) : null, dBias: tb ? upload(tb) : null };
    }
    if (st.kind !== 'linear' && st.kind !== 'dot') return null;
    const w = unb64(q.w, (x) => new Int8Array(x))!;
    let dW = upload(w);
    if (q.w_layout === 1) { const t = alloc(w.byteLength); check(b, b.transposeI8(ctx, dW, q.K, q.N, t), 'b200q_transpose_i8'); check(b, b.sync(ctx), 'b200q_sync'); check(b, b.free(ctx, dW), 'b200q_free'); dW = t; }
    if (st.kind === 'dot') return { dW, dWs: null, dBias: null };
    const bias = unb64(q.bias, (x) => new Float32Array(x));
    return { dW, dWs: upload(unb64(q.w_scales, (x) => new Float32Array(x))!), dBias: bias ? upload(bias) : null };
  });
  return {
    inputs: p.args.length, outputs: p.returns.length, steps: [],
    describe: () => p.steps.map((s) => s.kind).join('\n'),
    execute(bind, c, args) {
      p.args.forEach((a, i) => check(bind, bind.upload(c, buf.get(a.id), args[i], args[i].byteLength), 'b200q_upload'));
      p.steps.forEach((st, i) => {
        if (st.kind === 'const') return;
        const q = st.params as Record<string, any>, x = buf.get(st.ins[0]), y = buf.get(st.out.id), d = dev[i];
        if (st.kind === 'conv') runConv(bind, c, x, buf.get(st.ins[1]), y, { ...(q as ConvParams), kernelShape: q.kernel_shape, zpIn: q.zp_in, zpKer: q.zp_ker });
        else if (st.kind === 'shift') check(bind, bind.shiftU8ToI8(c, x, q.n, y), 'b200q_shift_u8_to_i8');
        else if (st.kind === 'dot') check(bind, bind.int8GemmI32(c, x, d!.dW, q.M, q.N, q.K, q.zp_a, q.zp_w, y), 'b200q_int8_gemm_i32');
        else if (st.kind === 'tail') {
          if (d!.dWs) check(bind, bind.epilogue(c, x, q.M, q.N, null, d!.dWs, d!.dBias, ACT[q.act as Act], y), 'b200q_epilogue');
          else check(bind, bind.epilogueTensorScale(c, x, q.M, q.N, q.tensor_scale, d!.dBias, ACT[q.act as Act], y), 'b200q_epilogue_tensor_scale');
        } else if (st.kind === 'quantize_static') check(bind, bind.quantizeStatic(c, x, elems.get(st.ins[0])!, q.scale, q.zero_point, q.kind, y), 'b200q_quantize_static');
        else if (st.kind === 'quantize_token') check(bind, bind.quantizePerToken(c, x, q.M, q.K, y, scales.get(st.out.id), -127, 127), 'b200q_quantize_per_token');
        else if (st.kind === 'dequantize_static') check(bind, bind.dequantizeStatic(c, x, q.kind, elems.get(st.ins[0])!, q.scale, q.zero_point, y), 'b200q_dequantize_static');
        else if (q.requant_scale !== null) check(bind, bind.int8LinearRequantStatic(c, x, null, d!.dW, d!.dWs, d!.dBias, ACT[q.act as Act], q.M, q.N, q.K, q.requant_scale, y), 'b200q_int8_linear_requant_static');
        else check(bind, bind.int8Linear(c, x, q.a_dynamic ? scales.get(st.ins[0]) : null, d!.dW, d!.dWs, d!.dBias, ACT[q.act as Act], q.M, q.N, q.K, y), 'b200q_int8_linear');
      });
      check(bind, bind.sync(c), 'b200q_sync');
      p.returns.forEach((id, i) => { const a = args[p.args.length + i]; check(bind, bind.download(c, a, buf.get(id), a.byteLength), 'b200q_download'); });
    },
  };
}
