"""Calibration with the observed tensors left on the device: min/max, percentile (0.999) and entropy modes.

Mirrors ``ValueObserver`` / ``HistogramCollector`` / ``CalibrationResult.getQuantParams`` of the reference
(src/compiler/analysis/calibration.ts:11-39, 41-186, 246-268): an observer keeps the running minimum and maximum of
everything it is shown and, in the histogram modes, a 2048-bin histogram whose range widens (with the old counts
re-bucketed at their bin centres) whenever a batch falls outside it; the quantization parameters follow from
``QuantizationParams.fromRange`` (src/compiler/ir/graph/quantization_types.ts:248-263) applied to the observed range,
to +-(the 0.999 percentile) or to +-(the clipping point of least KL divergence).  The passes over the data - the
reductions and the binning - run on the GPU; what remains is arithmetic on two numbers or on 2048 counts, done on the
host in binary64 as the reference does it (the two threshold searches by the library's own host routines).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

import ctypes as C

from . import _lib
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
    zp = cmin - mn / scale
    if zp != zp:     # the reference ends up with a NaN zero point here (Math.round(NaN)); nothing sensible follows from one
        raise ValueError(f"from_range: the range [{mn}, {mx}] has no asymmetric zero point (not a number)")
    zp = max(cmin, min(cmax, zp)) if zp in (math.inf, -math.inf) else _js_round(zp)
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


class HistogramState:
    """The fields and host-side steps of ``HistogramCollector`` (calibration.ts:41-186); binning the data itself is
    left to the caller (:class:`DeviceHistogramObserver` does it on the GPU, :meth:`add_host` with numpy for data that
    is on the host anyway)."""

    def __init__(self, num_bins: int = 2048):
        self.num_bins = num_bins
        self.bins = np.zeros(num_bins, np.float64)
        self.range_min = 0.0
        self.range_max = 0.0
        self.initialized = False
        self.total_count = 0

    def prepare(self, batch_min: float, batch_max: float) -> bool:
        """What ``update`` does before it bins a batch whose NaN-ignoring minimum and maximum are given: sets the range
        from the first batch (:81-90), returns False if the range is empty (:62-63), widens the range and re-buckets the
        old counts if the batch falls outside it (:92-120).  True means: bin the batch over [range_min, range_max]."""
        if not self.initialized:
            mn, mx = batch_min, batch_max
            if mn == mx:
                mx = mn + 1
            self.range_min, self.range_max, self.initialized = mn, mx, True
        if not (self.range_max - self.range_min > 0):
            return False
        if batch_min < self.range_min or batch_max > self.range_max:
            new_min, new_max = min(self.range_min, batch_min), max(self.range_max, batch_max)
            old_bins, old_min = self.bins.copy(), self.range_min
            old_range = self.range_max - self.range_min
            self.range_min, self.range_max = new_min, new_max
            with np.errstate(all="ignore"):
                new_scale = np.float64(self.num_bins) / np.float64(new_max - new_min)
                self.bins[:] = 0.0
                if old_range > 0:
                    width = old_range / self.num_bins
                    for i in np.nonzero(old_bins)[0]:
                        center = old_min + (i + 0.5) * width
                        idx = np.floor((center - new_min) * new_scale)
                        if idx == idx:                                   # a NaN index stores nowhere
                            self.bins[int(min(self.num_bins - 1, idx))] += old_bins[i]
        return True

    def add_host(self, data: np.ndarray) -> None:
        """``update`` for data on the host (numpy does the binning, in the same binary64 arithmetic)."""
        d = np.asarray(data, np.float64).reshape(-1)
        finite_cmp = d[~np.isnan(d)]
        mn = float(finite_cmp.min()) if finite_cmp.size else math.inf
        mx = float(finite_cmp.max()) if finite_cmp.size else -math.inf
        if not self.prepare(mn, mx):
            return
        with np.errstate(all="ignore"):
            raw = (d - self.range_min) * (np.float64(self.num_bins) / np.float64(self.range_max - self.range_min))
        raw = raw[~np.isnan(raw)]
        idx = np.minimum(self.num_bins - 1, np.floor(raw)).astype(np.int64)
        np.add.at(self.bins, idx, 1.0)
        self.total_count += d.size

    def percentile_threshold(self, percentile: float) -> float:
        out = C.c_double()
        b = np.ascontiguousarray(self.bins, np.float64)
        _lib.check(_lib.lib().b200q_histogram_percentile_threshold(b.ctypes.data, self.num_bins, float(self.total_count), self.range_min,
                                                                   self.range_max, percentile, C.byref(out)), "b200q_histogram_percentile_threshold")
        return out.value

    def entropy_threshold(self, num_quant_bins: int) -> float:
        out = C.c_double()
        b = np.ascontiguousarray(self.bins, np.float64)
        _lib.check(_lib.lib().b200q_histogram_entropy_threshold(b.ctypes.data, self.num_bins, float(self.total_count), self.range_min,
                                                                self.range_max, num_quant_bins, C.byref(out)), "b200q_histogram_entropy_threshold")
        return out.value


def histogram_quant_params(mode: str, observed: Tuple[float, float], hist: HistogramState, symmetric: bool = True, unsigned: bool = False,
                           num_bits: int = 8) -> QuantParams:
    """``CalibrationResult.getQuantParams`` (calibration.ts:246-268) for the modes 'minmax', 'percentile' and 'entropy'."""
    mn, mx = observed
    if mode == "percentile" and symmetric:
        hi = hist.percentile_threshold(0.999)
        return from_range(-hi, hi, True, unsigned, num_bits)
    if mode == "entropy" and symmetric:
        t = hist.entropy_threshold(256 if unsigned else 255)
        return from_range(-t, t, True, unsigned, num_bits)
    if mode not in ("minmax", "percentile", "entropy"):
        raise ValueError(f"unknown calibration mode {mode!r}")
    return from_range(mn, mx, symmetric, unsigned, num_bits)


class DeviceHistogramObserver(DeviceObserver):
    """:class:`DeviceObserver` with the histogram of the percentile and entropy modes: per batch one reduction (the
    batch's range, needed on the host to decide whether the histogram has to widen) and one binning pass, both on the
    GPU."""

    def __init__(self, ctx: Context, mode: str = "percentile", num_bins: int = 2048):
        super().__init__(ctx)
        self.mode = mode
        self.hist = HistogramState(num_bins)
        self._batch = ctx.empty((2,), np.float32)
        self._bins = ctx.empty((num_bins,), np.uint64)

    def update(self, x, n: int) -> None:
        super().update(x, n)
        ctx = self.ctx
        ctx.observer_reset(self._batch)
        ctx.observe_minmax(x, n, self._batch)
        ctx.sync()
        bmin, bmax = (float(v) for v in self._batch.download())
        if not self.hist.prepare(bmin, bmax):
            return
        self._bins.fill_bytes(0)
        ctx.histogram_f32(x, n, self.hist.range_min, self.hist.range_max, self.hist.num_bins, self._bins)
        ctx.sync()
        self.hist.bins += self._bins.download().astype(np.float64)
        self.hist.total_count += n

    def quant_params(self, symmetric: bool = True, unsigned: bool = False, num_bits: int = 8) -> Optional[QuantParams]:
        r = self.range()
        return None if r is None else histogram_quant_params(self.mode, r, self.hist, symmetric, unsigned, num_bits)
