// RuntimeModuleLike (src/compiler/support/config_types.ts:58-66) over libb200q.so.
// The graph is matched once at construction into a list of native steps (see planGraph,
// whose rules are the ones of mlfw_b200/backend.py: plan_function); run() marshals typed arrays
// or {data, shape, dtype} tensors (both argument forms of src/runtime/runtime.ts:242-250) into
// one host-buffer call per step.
import { loadB200Q, check } from './binding.js';
import { planGraph } from './plan.js';               // the matcher; a transliteration of backend.py:plan_function

import type { RuntimeModuleLike } from '../../compiler/support/config_types.js';
import type { GraphModule } from '../../compiler/ir/graph/module.js';
import type { B200Options } from './target.js';

type TensorArg = ArrayBufferView | { data: ArrayBufferView; shape: readonly number[]; dtype: string };
const view = (t: TensorArg): ArrayBufferView => (ArrayBuffer.isView(t) ? t : t.data);

export class B200RuntimeModule implements RuntimeModuleLike {
  private b; private ctx: unknown; private plans;
  constructor(module: GraphModule, options: B200Options) {
    this.b = loadB200Q(options.library ?? 'libb200q.so');
    const out: [unknown] = [null];
    check(this.b, this.b.create(options.device ?? 0, out), 'b200q_create');   // no GPU: throws, there is no fallback
    this.ctx = out[0];
    this.plans = planGraph(module, options, this.b, this.ctx);                 // uploads weights, scale vectors, biases once
  }
  run(funcName: string, ...args: TensorArg[]): void {
    const plan = this.plans.get(funcName);
    if (!plan) throw new Error(`b200: no function named ${funcName}`);
    if (args.length !== plan.inputs + plan.outputs) throw new Error(`b200: ${funcName} takes ${plan.inputs} tensors and returns ${plan.outputs}`);
    plan.execute(this.b, this.ctx, args.map(view));                            // device steps, then one sync
  }
  runAsync(funcName: string, ...args: TensorArg[]): Promise<void> { return Promise.resolve(this.run(funcName, ...args)); }
  isAsync(): boolean { return false; }
  getKernelSource(funcName: string): string | null { return this.plans.has(funcName) ? this.plans.get(funcName).describe() : null; }
  getKernelMetadata(funcName: string): Record<string, unknown> | null {
    const p = this.plans.get(funcName);
    return p ? { kind: 'b200', inputs: p.inputs, outputs: p.outputs, steps: p.steps.length } : null;
  }
  listKernels(): string[] { return [...this.plans.keys()]; }
  release(): void { if (this.ctx) { this.b.destroy(this.ctx); this.ctx = null; } }
}
