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
