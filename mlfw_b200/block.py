"""A pre-norm transformer block with int8 linears, run as a sequence of library calls on one GPU.

Mirrors ``TransformerEncoderLayer`` with ``normFirst`` of the reference (src/nn/modules/transformer.ts:144-152,
built by the GPT-2 fixture tests/_utils/gpt2_model.js:5 with a causal mask and GELU) after its quantization pass has
turned the four ``Linear`` modules into quantize -> quantized_dot -> per-channel tail chains
(src/compiler/passes/quantization/quantization_pass.ts:390-459), with dynamic per-token activation scales:

    n1 = LayerNorm1(h)                                   codes + scales come straight out of the LayerNorm kernel
    q, k, v = n1 Wq^T + bq, n1 Wk^T + bk, n1 Wv^T + bv   one int8 GEMM over the stacked [3D, D] weight
    a = attention(q, k, v)                               f32, causal, scale 1/sqrt(D/H)
    x = h + (a Wo^T + bo)
    y = x + (gelu(LayerNorm2(x) W1^T + b1) W2^T + b2)    the residual sum x is formed inside the LayerNorm2 launch; the
                                                         requantization of W2's input starts in W1's epilogue

Weights are quantized per output channel on the device when the block is built and stay resident.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np

from .device import Context, DeviceBuffer, W_NK


@dataclass
class QuantLinear:
    """int8 weight [N, K] (K-major), per-channel scales, bias; resident on the device."""
    N: int
    K: int
    w: DeviceBuffer
    scales: DeviceBuffer
    bias: Optional[DeviceBuffer]

    @staticmethod
    def from_float(ctx: Context, weight: np.ndarray, bias: Optional[np.ndarray]) -> "QuantLinear":
        """``weight`` is the reference's ``Linear.weight`` layout [out, in] (src/nn/modules/linear.ts:18)."""
        weight = np.ascontiguousarray(weight, np.float32)
        N, K = weight.shape
        dw = ctx.to_device(weight)
        qw = ctx.empty((N, K), np.int8)
        sc = ctx.empty((N,), np.float32)
        ctx.quantize_weights_per_channel(dw, N, K, W_NK, qw, sc)
        ctx.sync()
        dw.free()
        return QuantLinear(N, K, qw, sc, ctx.to_device(np.ascontiguousarray(bias, np.float32)) if bias is not None else None)

    def state(self):
        """This linear as it goes into an ``mlfw-ckpt-v1`` checkpoint (:mod:`mlfw_b200.checkpoint`)."""
        from .checkpoint import quantized_linear_state
        return quantized_linear_state(self.w.download(), self.scales.download(), self.bias.download() if self.bias is not None else None)

    @staticmethod
    def from_state(ctx: Context, st) -> "QuantLinear":
        """Rebuild from :meth:`state` without running the quantization again: the codes and scales are uploaded as they are."""
        wq = np.ascontiguousarray(st["weight_q"].data, np.int8)
        N, K = wq.shape
        bias = st.get("bias")
        return QuantLinear(N, K, ctx.to_device(wq), ctx.to_device(np.ascontiguousarray(st["weight_scale"].data, np.float32)),
                           ctx.to_device(np.ascontiguousarray(bias.data, np.float32)) if bias is not None else None)


class GPTBlock:
    """One block for activations [B*S, D]; ``forward`` enqueues everything on the context's stream."""

    def __init__(self, ctx: Context, D: int, H: int, FF: int, params: Dict[str, np.ndarray], eps: float = 1e-5,
                 activation: str = "gelu_sigmoid"):
        assert D % H == 0 and D // H == 64, "the attention kernel is built for a head dimension of 64"
        self.ctx, self.D, self.H, self.FF, self.eps, self.activation = ctx, D, H, FF, eps, activation
        f32 = lambda name: ctx.to_device(np.ascontiguousarray(params[name], np.float32))
        self.g1, self.b1, self.g2, self.b2 = f32("ln1_gamma"), f32("ln1_beta"), f32("ln2_gamma"), f32("ln2_beta")
        wqkv = np.concatenate([params["wq"], params["wk"], params["wv"]], axis=0)
        bqkv = np.concatenate([params["bq"], params["bk"], params["bv"]], axis=0)
        self.qkv = QuantLinear.from_float(ctx, wqkv, bqkv)
        self.wo = QuantLinear.from_float(ctx, params["wo"], params["bo"])
        self.fc1 = QuantLinear.from_float(ctx, params["w1"], params["b1"])
        self.fc2 = QuantLinear.from_float(ctx, params["w2"], params["b2"])
        self._bufs: Dict[str, DeviceBuffer] = {}
        self._M = -1

    def _reserve(self, M: int) -> Dict[str, DeviceBuffer]:
        if M != self._M:
            c, D, FF = self.ctx, self.D, self.FF
            self._bufs = {
                "n1_q": c.empty((M, D), np.int8), "n1_s": c.empty((M,), np.float32), "qkv": c.empty((M, 3 * D), np.float32),
                "attn": c.empty((M, D), np.float32), "o": c.empty((M, D), np.float32), "x": c.empty((M, D), np.float32),
                "n2_q": c.empty((M, D), np.int8), "n2_s": c.empty((M,), np.float32), "f1": c.empty((M, FF), np.float32),
                "f1_q": c.empty((M, FF), np.int8), "f1_s": c.empty((M,), np.float32), "f2": c.empty((M, D), np.float32),
            }
            self._M = M
        return self._bufs

    def forward(self, h: DeviceBuffer, B: int, S: int, out: DeviceBuffer, causal: bool = True) -> Dict[str, DeviceBuffer]:
        """h, out: f32 [B*S, D].  Returns the intermediate buffers (reused by the next call with the same size)."""
        c, D, H, FF = self.ctx, self.D, self.H, self.FF
        M = B * S
        t = self._reserve(M)
        c.layernorm_quantize(h, None, self.g1, self.b1, self.eps, M, D, None, None, t["n1_q"], t["n1_s"])
        c.int8_linear(t["n1_q"], t["n1_s"], self.qkv.w, self.qkv.scales, self.qkv.bias, "none", M, 3 * D, D, t["qkv"])
        base = t["qkv"].ptr
        c.sdpa_f32(base, base + D * 4, base + 2 * D * 4, 3 * D, 3 * D, 3 * D, B, H, S, 64, 1.0 / np.sqrt(64.0), causal, t["attn"], D)
        c.linear_f32(t["attn"], self.wo.w, self.wo.scales, self.wo.bias, "none", M, D, D, t["o"])
        c.layernorm_quantize(t["o"], h, self.g2, self.b2, self.eps, M, D, t["x"], None, t["n2_q"], t["n2_s"])
        # FC1 with the requantization of FC2's input behind it: the rows' ranges come out of FC1's epilogue, one pass encodes
        c.int8_linear_f32_requant_token(t["n2_q"], t["n2_s"], self.fc1.w, self.fc1.scales, self.fc1.bias, self.activation, M, FF, D,
                                        t["f1"], t["f1_q"], t["f1_s"])
        c.int8_linear(t["f1_q"], t["f1_s"], self.fc2.w, self.fc2.scales, self.fc2.bias, "none", M, D, FF, t["f2"])
        c.add_f32(t["x"], t["f2"], M * D, out)
        return t


def random_block_params(D: int, FF: int, seed: int = 0, std: float = 0.02) -> Dict[str, np.ndarray]:
    """Weights ~N(0, std), biases ~N(0, std), LayerNorm gamma 1 / beta 0 (the shapes of the GPT-2 fixture)."""
    rng = np.random.default_rng(seed)
    n = lambda *shape: (rng.standard_normal(shape) * std).astype(np.float32)
    return {
        "ln1_gamma": np.ones(D, np.float32), "ln1_beta": np.zeros(D, np.float32),
        "ln2_gamma": np.ones(D, np.float32), "ln2_beta": np.zeros(D, np.float32),
        "wq": n(D, D), "wk": n(D, D), "wv": n(D, D), "wo": n(D, D), "bq": n(D), "bk": n(D), "bv": n(D), "bo": n(D),
        "w1": n(FF, D), "b1": n(FF), "w2": n(D, FF), "b2": n(D),
    }
