// B200Target(): a TargetFeatures whose EXTERNAL_COMPILER hands the post-pass graph to
// libb200q.so.  Registration uses only seams the reference already has
// (src/compiler/support/target.ts:20-55, TargetAttr.EXTERNAL_COMPILER consumed at
// src/compiler/pipeline/compiler.ts:297-329; precedent src/backend/terac/target.ts:16-38),
// so src/nn, src/tensor and the quantization and fusion passes run unchanged:
//
//   const compiled = compile(model, [x], { target: B200Target(), foldWeights: true,
//                                          quantization: { enabled: true, scheme: 'per_channel',
//                                                          quantizableOps: new Set(['dot']) } });
//
// kind 'accelerator' is declared by the reference and unused (target.ts:3-9); it is not a GPU kind
// for calibrate_exec.ts:79-81, so a precomputed `quantization.calibration` object keeps working.
import { TargetFeatures, TargetKind } from '../../compiler/support/target.js';
import { TargetAttr, targetAttr } from '../../compiler/support/target_attrs.js';
import { B200RuntimeModule } from './runtime_module.js';

import type { CompilerConfig, RuntimeModuleLike } from '../../compiler/support/config_types.js';
import type { GraphModule } from '../../compiler/ir/graph/module.js';

export const B200_OPTIONS = 'b200Options';

export type B200Options = {
  library?: string;                                   // path of libb200q.so
  device?: number;                                    // CUDA ordinal
  activationQuant?: 'static' | 'per_token_dynamic';   // 'static' reproduces the reference's scales
};

export function compileWithB200(module: GraphModule, config: CompilerConfig): RuntimeModuleLike {
  const options = targetAttr<B200Options>(config.target, B200_OPTIONS) || {};
  return new B200RuntimeModule(module, options);     // throws on any op outside the graph contract
}

export function B200Target(options: B200Options = {}): TargetFeatures {
  return new TargetFeatures({
    kind: TargetKind.ACCELERATOR,
    name: 'b200_int8',
    supportsInt8: true,                               // QuantizationPass bails without it (quantization_pass.ts:94)
    supportsConstBuffers: true,
    attrs: {
      [TargetAttr.FUSION]: { enabled: false },        // the contract then arrives as a flat op list
      [TargetAttr.EXTERNAL_COMPILER]: compileWithB200,
      [B200_OPTIONS]: { activationQuant: 'static', device: 0, ...options },
    },
  });
}
