"""Calibration (min/max mode): the host restatement of ``fromRange`` against the oracle and the reference's known
answers, and the device observer against the oracle's observer."""
import numpy as np
import pytest

from mlfw_b200.calibration import from_range


def test_from_range_known_answers():
    # tests/compiler/passes/quantization/params.test.js:6-23, 90-119: symmetric scale = absMax/127, default activation 6/127
    p = from_range(-6, 6)
    assert p.scale == 6 / 127 and p.zero_point == 0 and p.clamp == (-127, 127)
    assert from_range(-1.5, 3.0).scale == 3.0 / 127
    # params.test.js:26-41: asymmetric scale = range/255, zero point clamped; ui8 [0, 255]
    q = from_range(-1.0, 3.0, symmetric=False)
    assert q.scale == 4.0 / 255 and q.clamp == (-128, 127) and -128 <= q.zero_point <= 127
    assert from_range(0.0, 2.0, symmetric=False, unsigned=True).clamp == (0, 255)
    assert from_range(0.0, 0.0).scale == 1e-10


def test_from_range_matches_oracle(orc):
    rng = np.random.default_rng(0)
    cases = [(-6.0, 6.0), (0.0, 0.0), (2.0, 2.0), (-0.3, 0.1), (1e-30, 2e-30), (-1e30, 5.0)]
    cases += [tuple(float(v) for v in sorted(rng.standard_normal(2) * 10.0 ** rng.integers(-5, 5))) for _ in range(200)]
    for mn, mx in cases:
        s, zp = orc.from_range(mn, mx)
        p = from_range(mn, mx)
        assert p.scale == s and p.zero_point == zp
        s, zp = orc.from_range(mn, mx, scheme=orc.SCHEME_ASYM)
        p = from_range(mn, mx, symmetric=False)
        assert p.scale == s and p.zero_point == zp


@pytest.mark.gpu
def test_device_observer_matches_oracle(orc):
    import mlfw_b200
    from mlfw_b200.calibration import DeviceObserver
    rng = np.random.default_rng(1)
    with mlfw_b200.Context(0) as ctx:
        obs = DeviceObserver(ctx)
        assert obs.range() is None and obs.quant_params() is None
        batches = [rng.standard_normal(100003).astype(np.float32) * 3, rng.standard_normal(7).astype(np.float32) - 20,
                   np.array([np.nan, 1.0, -np.nan, 25.5], np.float32), rng.standard_normal((64, 768)).astype(np.float32).ravel()]
        for b in batches:
            obs.update(ctx.to_device(b), b.size)
        mn, mx = obs.range()
        ref = orc.minmax_observe(batches)
        assert (mn, mx) == ref
        assert obs.quant_params().scale == orc.from_range(*ref)[0]
        # a view that starts 4 bytes into an allocation (scalar path), an all-NaN batch, and infinities
        obs2 = DeviceObserver(ctx)
        buf = ctx.to_device(batches[0])
        obs2.update(buf.ptr + 4, batches[0].size - 1)
        obs2.update(ctx.to_device(np.full(9, np.nan, np.float32)), 9)
        assert obs2.range() == orc.minmax_observe([batches[0][1:]])
        obs2.update(ctx.to_device(np.array([np.inf, -np.inf, 0.0, -0.0], np.float32)), 4)
        assert obs2.range() == (-np.inf, np.inf)
        # only negative values, then only -0.0 / +0.0
        obs3 = DeviceObserver(ctx)
        obs3.update(ctx.to_device(np.array([-3.0, -1.5, -2.0, -8.0, -1.25], np.float32)), 5)
        assert obs3.range() == (-8.0, -1.25)
        obs3.update(ctx.to_device(np.array([-0.0, 0.0, -0.0, 0.0], np.float32)), 4)
        assert obs3.range() == (-8.0, 0.0)
        ctx.check_status()


# ------------------------------------------------------------------ histogram modes (percentile, entropy)
def _batches(seed=3):
    rng = np.random.default_rng(seed)
    out = [rng.standard_normal(5000).astype(np.float32), (rng.standard_normal(3000) * 3 + 1).astype(np.float32),   # widens the range
           rng.standard_normal(2000).astype(np.float32) * 0.1]
    out[1][7] = np.nan
    return out


def test_histogram_state_follows_the_line_by_line_port():
    """The host mirror (numpy binning, library threshold routines) against the pure-Python port of HistogramCollector:
    same range, same counts after widening and re-bucketing, same percentile and entropy thresholds, same parameters."""
    from oracle import jsport as js
    from mlfw_b200.calibration import HistogramState, histogram_quant_params
    h, ref = HistogramState(256), js.HistogramCollector(256)      # 256 bins keep the pure-Python entropy search short
    for b in _batches():
        h.add_host(b)
        ref.update([float(v) for v in b])
        assert (h.range_min, h.range_max, h.total_count) == (ref.range_min, ref.range_max, ref.total_count)
        assert (h.bins == np.array(ref.bins)).all()
    assert h.percentile_threshold(0.999) == ref.compute_percentile_threshold(0.999)
    assert h.percentile_threshold(0.5) == ref.compute_percentile_threshold(0.5)
    for nq in (32, 64, 255):
        assert h.entropy_threshold(nq) == ref.compute_entropy_threshold(nq)
    obs = (-9.0, 11.0)
    p = histogram_quant_params("percentile", obs, h)
    assert p.scale == ref.compute_percentile_threshold(0.999) / 127 and p.zero_point == 0
    assert histogram_quant_params("entropy", obs, h).scale == ref.compute_entropy_threshold(255) / 127
    assert histogram_quant_params("entropy", obs, h, unsigned=True).scale == ref.compute_entropy_threshold(256) / 127
    assert histogram_quant_params("percentile", obs, h, symmetric=False).scale == 20.0 / 255       # asymmetric: the observed range
    assert histogram_quant_params("minmax", obs, h).scale == 11.0 / 127
    # degenerate inputs: a constant first batch (range widened by one), an all-NaN batch, an empty histogram
    h2, r2 = HistogramState(64), js.HistogramCollector(64)
    for b in ([2.5] * 10, [float("nan")] * 4, [2.5, 3.0, 9.0]):
        h2.add_host(np.array(b, np.float32)); r2.update([float(np.float32(v)) for v in b])
        assert (h2.range_min, h2.range_max, h2.total_count) == (r2.range_min, r2.range_max, r2.total_count) and (h2.bins == np.array(r2.bins)).all()
    assert HistogramState(64).entropy_threshold(16) == js.HistogramCollector(64).compute_entropy_threshold(16) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["percentile", "entropy"])
def test_device_histogram_observer_matches_the_host_mirror(mode):
    import mlfw_b200
    from mlfw_b200.calibration import DeviceHistogramObserver, HistogramState, histogram_quant_params
    rng = np.random.default_rng(11)
    batches = _batches(5) + [rng.standard_normal(300000).astype(np.float32) * 2, np.array([40.0, -35.0, np.nan, 0.0], np.float32)]
    with mlfw_b200.Context(0) as ctx:
        obs = DeviceHistogramObserver(ctx, mode)
        host = HistogramState()
        for b in batches:
            obs.update(ctx.to_device(b), b.size)
            host.add_host(b)
            assert (obs.hist.range_min, obs.hist.range_max, obs.hist.total_count) == (host.range_min, host.range_max, host.total_count)
            assert (obs.hist.bins == host.bins).all()
        allv = np.concatenate(batches)
        fin = allv[~np.isnan(allv)]
        assert obs.range() == (float(fin.min()), float(fin.max()))
        p = obs.quant_params()
        q = histogram_quant_params(mode, obs.range(), host)
        assert p == q and 0 < p.scale < max(abs(fin.min()), fin.max()) / 127     # clipped inside the observed range
        ctx.check_status()
