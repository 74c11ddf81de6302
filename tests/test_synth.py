"""The product's numpy data generators agree with the oracle's restatement of the reference generators."""
import numpy as np

from mlfw_b200 import synth


def test_uniform_stream_is_mulberry32(orc):
    for seed in (0, 1, 12345, 0x9E3779B9, synth.tensor_seed(3, 7)):
        assert (synth.mulberry32(seed, 1000) == orc.rng_uniform(seed, 1000)).all()


def test_normal_and_uniform_tensors(orc):
    a = synth.normal(5, (33, 7), 0.0, 0.02)
    b = orc.normal_f32(5, (33, 7), 0.0, 0.02)
    assert np.abs(a - b).max() <= 2e-9            # libm differences of an ulp at most
    assert (synth.uniform(9, (100,), -0.1, 0.1) == orc.uniform_f32(9, (100,), -0.1, 0.1)).all()
    assert (synth.randint_i8(4, (1000,)) == orc.randint_i8(4, (1000,))).all()
    w = synth.randint_i8(4, (100000,))
    assert w.min() == -127 and w.max() == 127


def test_outliers():
    x = synth.normal(1, (256, 512))
    y = synth.with_outliers(x, 2, 3)
    frac = (x != y).mean()
    assert 0.0005 < frac < 0.002
    assert np.abs(y[x != y]).std() > 10
