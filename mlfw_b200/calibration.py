"""Min/max calibration with the observed tensors left on the device.

Mirrors ``ValueObserver`` / ``CalibrationResult.getQuantParams`` of the reference in min/max mode
(src/compiler/analysis/calibration.ts:11-39, 246-268): an observer keeps the running minimum and maximum of everything
it is shown; the quantization parameters follow from ``QuantizationParams.fromRange``
(src/compiler/ir/graph/quantization_types.ts:248-263).  Only the reduction runs on the GPU; the handful of scalar
operations of ``from_range`` are host arithmetic in binary64, as in the reference.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

from .device import Context


@dataclass
class QuantParams:
    scale: float
    zero_point: int
    clamp: Tuple[int, int]


def _js_round(x: float) -> float:
    """Math.round: nearest integer, ties toward +infinity."""
    r = math.floor(x)
    return r + 1.0 if x - r >= 0.5 else r


def from_range(mn: float, mx: float, symmetric: bool = True, unsigned: bool = False, num_bits: int = 8) -> QuantParams:
    """QuantizationParams.fromRange (quantization_types.ts:248-263)."""
    if symmetric:
        bound = 2 ** (num_bits - 1) - 1
        scale = max(abs(mn), abs(mx)) / bound or 1e-10
        if scale != scale:   # NaN is falsy in JavaScript too
            scale = 1e-10
        return QuantParams(scale, 0, (-bound, bound))
    cmin, cmax = (0, 2 ** num_bits - 1) if unsigned else (-(2 ** (num_bits - 1)), 2 ** (num_bits - 1) - 1)
    rng = (mx - mn) or 1e-10
    scale = rng / (cmax - cmin)
    zp = _js_round(cmin - mn / scale)
    return QuantParams(scale, int(max(cmin, min(cmax, zp))), (cmin, cmax))


class DeviceObserver:
    """Running min / max of the tensors passed to :meth:`update` (device pointers), NaN ignored."""

    def __init__(self, ctx: Context):
        self.ctx = ctx
        self.state = ctx.empty((2,), np.float32)
        self.count = 0
        ctx.observer_reset(self.state)

    def update(self, x, n: int) -> None:
        self.ctx.observe_minmax(x, n, self.state)
        self.count += n

    def range(self) -> Optional[Tuple[float, float]]:
        """(min, max) as binary64 numbers, or None when nothing was observed (``getRange``)."""
        if self.count == 0:
            return None
        self.ctx.sync()
        mn, mx = self.state.download()
        return float(mn), float(mx)

    def quant_params(self, symmetric: bool = True, unsigned: bool = False, num_bits: int = 8) -> Optional[QuantParams]:
        r = self.range()
        return None if r is None else from_range(r[0], r[1], symmetric, unsigned, num_bits)
