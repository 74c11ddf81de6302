// Registration of the B200 backend with the reference's remaining registries.  target.ts covers the whole-module seam
// (TargetAttr.EXTERNAL_COMPILER); this file covers the other two the reference offers:
//
//   * the runtime backend registry - registerBackend(kind, {instantiate, runSync, runAsync, isAsync})
//     (src/runtime/backend_registry.ts:14-36, looked up by kernel.metadata.kind in src/runtime/runtime.ts:212-220):
//     a CompiledKernel whose metadata.kind is 'b200' carries a native program (the step list planGraph makes, as
//     JSON in `source`); instantiate() turns it into a plan bound to a device context, runSync() marshals the typed
//     arrays it is given (arguments, then outputs, then constant buffers: runtime.ts:239-259) into the plan;
//   * the eager dispatcher - four ops under DispatchKey.CUSTOM_1 (src/dispatcher/dispatcher.ts:81-86,
//     library.ts:30-59; CUSTOM_1..3 are free, dispatch_key.ts:8-10), entered with withB200(() => ...), so that
//     src/tensor users reach the kernels without a new device name (the device -> key table is a frozen literal,
//     dispatch_key.ts:36-43).
//
// Source only in this repository (no JavaScript engine in the build image); every call below goes through the same C
// ABI the Python host and the tests use.
import { registerBackend } from '../../runtime/backend_registry.js';
import { Library } from '../../dispatcher/library.js';
import { DispatchKey, DispatchKeySet } from '../../dispatcher/dispatch_key.js';
import { withIncludedKeys } from '../../dispatcher/guard.js';
import { wrapResult, tensorToContiguous } from '../../dispatcher/jit_dispatch.js';
import { loadB200Q, check } from './binding.js';
import { planFromProgram } from './plan.js';

import type { RuntimeKernel } from '../../runtime/runtime.js';
import type { Tensor } from '../../tensor/core/tensor.js';
import type { B200QBinding } from './binding.js';
import type { FunctionPlan } from './plan.js';

export const B200_KIND = 'b200';
const ACT = { none: 0, relu: 1, gelu_sigmoid: 2, gelu_tanh: 3, silu: 4 } as const;

type Session = { b: B200QBinding; ctx: unknown };
let session: Session | null = null;

/** One device context per process for the registry paths (the reference's CUDA runtime also owns a single device). */
export function b200Session(library = 'libb200q.so', device = 0): Session {
  if (session) return session;
  const b = loadB200Q(library);
  const out: [unknown] = [null];
  check(b, b.create(device, out), 'b200q_create');            // no GPU: throws - there is no fallback
  session = { b, ctx: out[0] };
  return session;
}

// ------------------------------------------------------------------------------------------ runtime backend kind
type B200Instance = { plan: FunctionPlan };

export function registerB200RuntimeBackend(library?: string, device?: number): void {
  registerBackend(B200_KIND, {
    instantiate(kernel: RuntimeKernel): B200Instance {
      const s = b200Session(library, device);
      // kernel.source is the native program: JSON of the steps with weights, scale vectors and biases as base64
      return { plan: planFromProgram(JSON.parse(kernel.source), s.b, s.ctx) };
    },
    runSync(instance: unknown, tensorArgs: readonly ArrayBufferView[]): void {
      const s = b200Session(library, device);
      (instance as B200Instance).plan.execute(s.b, s.ctx, tensorArgs as ArrayBufferView[]);
    },
    runAsync(instance: unknown, tensorArgs: readonly ArrayBufferView[]): Promise<void> {
      return Promise.resolve(this.runSync(instance, tensorArgs, null) as void);
    },
    isAsync(): boolean { return false; },                       // keeps compiled(x) synchronous (src/tracing/compile.ts:119-125)
  });
}

// ------------------------------------------------------------------------------------------ eager ops
const SCHEMAS = [
  'b200_quantize_per_token(Tensor x) -> (Tensor, Tensor)',                                   // codes i8 [M,K], scales f32 [M]
  'b200_dequantize_per_token(Tensor q, Tensor scales) -> Tensor',
  'b200_int8_linear(Tensor x, Tensor w_q, Tensor w_scales, Tensor bias, str activation) -> Tensor',   // f32 [M,K] x i8 [N,K] -> f32 [M,N]
  // i8 [N,C,H,W] x i8 [O,C/groups,KH,KW] -> i32 [N,O,OH,OW] (quantized_conv, src/compiler/ir/graph/ops/quantization.ts:156-190)
  'b200_quantized_conv2d(Tensor x, Tensor kernel, int[] strides, int[][] padding, int[] dilation, int groups, int zp_in, int zp_kernel) -> Tensor',
];

function onDevice<T>(s: Session, hostArrays: ArrayBufferView[], outBytes: number[], run: (ins: unknown[], outs: unknown[]) => void,
                     read: (outs: unknown[]) => T): T {
  const { b, ctx } = s;
  const alloc = (n: number) => { const p: [unknown] = [null]; check(b, b.alloc(ctx, n, p), 'b200q_alloc'); return p[0]; };
  const ins = hostArrays.map((a) => { const d = alloc(a.byteLength); check(b, b.upload(ctx, d, a, a.byteLength), 'b200q_upload'); return d; });
  const outs = outBytes.map(alloc);
  try {
    run(ins, outs);
    check(b, b.sync(ctx), 'b200q_sync');
    return read(outs);
  } finally {
    for (const d of [...ins, ...outs]) b.free(ctx, d);
  }
}

function quantizePerToken(_ks: unknown, x: Tensor): [Tensor, Tensor] {
  const s = b200Session();
  const [M, K] = x.shape;
  const host = tensorToContiguous(x) as Float32Array;
  return onDevice(s, [host], [M * K, M * 4],
    (i, o) => check(s.b, s.b.quantizePerToken(s.ctx, i[0], M, K, o[0], o[1], -127, 127), 'b200q_quantize_per_token'),
    (o) => {
      const q = new Int8Array(M * K), sc = new Float32Array(M);
      check(s.b, s.b.download(s.ctx, q, o[0], q.byteLength), 'b200q_download');
      check(s.b, s.b.download(s.ctx, sc, o[1], sc.byteLength), 'b200q_download');
      return [wrapResult(q, [M, K], 'i8', x.device), wrapResult(sc, [M], 'f32', x.device)];
    });
}

function dequantizePerToken(_ks: unknown, q: Tensor, scales: Tensor): Tensor {
  const s = b200Session();
  const [M, K] = q.shape;
  return onDevice(s, [tensorToContiguous(q) as Int8Array, tensorToContiguous(scales) as Float32Array], [M * K * 4],
    (i, o) => check(s.b, s.b.dequantizePerToken(s.ctx, i[0], i[1], M, K, o[0]), 'b200q_dequantize_per_token'),
    (o) => { const y = new Float32Array(M * K); check(s.b, s.b.download(s.ctx, y, o[0], y.byteLength), 'b200q_download'); return wrapResult(y, [M, K], 'f32', q.device); });
}

function int8Linear(_ks: unknown, x: Tensor, wq: Tensor, wScales: Tensor, bias: Tensor | null, activation: keyof typeof ACT): Tensor {
  const s = b200Session();
  const [M, K] = x.shape, N = wq.shape[0];
  if (!(activation in ACT)) throw new Error(`b200_int8_linear: unknown activation ${activation}`);
  const ins = [tensorToContiguous(x) as Float32Array, tensorToContiguous(wq) as Int8Array, tensorToContiguous(wScales) as Float32Array];
  if (bias) ins.push(tensorToContiguous(bias) as Float32Array);
  return onDevice(s, ins, [M * N * 4],
    (i, o) => check(s.b, s.b.linearF32(s.ctx, i[0], i[1], i[2], bias ? i[3] : null, ACT[activation], M, N, K, o[0]), 'b200q_linear_f32'),
    (o) => { const y = new Float32Array(M * N); check(s.b, s.b.download(s.ctx, y, o[0], y.byteLength), 'b200q_download'); return wrapResult(y, [M, N], 'f32', x.device); });
}

function quantizedConv2d(_ks: unknown, x: Tensor, ker: Tensor, strides: number[], padding: number[][], dilation: number[], groups: number,
                         zpIn: number, zpKer: number): Tensor {
  const s = b200Session();
  const [N, C, H, W] = x.shape, [O, , KH, KW] = ker.shape;
  const ext = (size: number, p: number[], k: number, st: number, d: number) => Math.floor((size + p[0] + p[1] - ((k - 1) * d + 1)) / st) + 1;   // ops/linalg.ts:236-246
  const OH = ext(H, padding[0], KH, strides[0], dilation[0]), OW = ext(W, padding[1], KW, strides[1], dilation[1]);
  return onDevice(s, [tensorToContiguous(x) as Int8Array, tensorToContiguous(ker) as Int8Array], [N * O * OH * OW * 4],
    (i, o) => check(s.b, s.b.quantizedConv2d(s.ctx, i[0], i[1], N, C, H, W, O, KH, KW, strides[0], strides[1], padding[0][0], padding[0][1],
                                             padding[1][0], padding[1][1], dilation[0], dilation[1], groups, zpIn, zpKer, 0, o[0]), 'b200q_quantized_conv2d'),
    (o) => { const y = new Int32Array(N * O * OH * OW); check(s.b, s.b.download(s.ctx, y, o[0], y.byteLength), 'b200q_download'); return wrapResult(y, [N, O, OH, OW], 'i32', x.device); });
}

let eagerRegistered = false;
export function registerB200EagerOps(): void {
  if (eagerRegistered) return;
  eagerRegistered = true;
  const defs = new Library('mlc', 'DEF');
  for (const schema of SCHEMAS) defs.def(schema);
  new Library('mlc', 'IMPL')
    .impl('b200_quantize_per_token', DispatchKey.CUSTOM_1, quantizePerToken)
    .impl('b200_dequantize_per_token', DispatchKey.CUSTOM_1, dequantizePerToken)
    .impl('b200_int8_linear', DispatchKey.CUSTOM_1, int8Linear)
    .impl('b200_quantized_conv2d', DispatchKey.CUSTOM_1, quantizedConv2d);
}

/** Runs fn with the CUSTOM_1 key included, so that dispatcher.callOp('b200_int8_linear', ...) reaches the kernels above. */
export function withB200<T>(fn: () => T): T {
  return withIncludedKeys(DispatchKeySet.fromKey(DispatchKey.CUSTOM_1), fn);
}

/** Everything at once: the runtime kind and the eager ops (the target object needs no registration). */
export function registerB200(library?: string, device?: number): void {
  registerB200RuntimeBackend(library, device);
  registerB200EagerOps();
}
