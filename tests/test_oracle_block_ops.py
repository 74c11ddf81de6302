"""The oracle's restatement of LayerNorm and attention against independent float64 numpy formulas.

The reference's own tests bound these operations only by tolerances (e.g. tests/tracing/compile.test.js compares
compiled and eager outputs to 1e-4), and store no vectors for them; the restatement is therefore pinned to the
mathematical definition here, to well inside the 1e-5 bar the device kernels are then held to against it.
"""
import numpy as np
import pytest


def test_layer_norm_matches_float64(orc):
    rng = np.random.default_rng(0)
    for M, D in [(7, 768), (3, 36), (5, 2048)]:
        x = (rng.standard_normal((M, D)) * 4 - 1).astype(np.float32)
        add = rng.standard_normal((M, D)).astype(np.float32)
        gamma = rng.uniform(0.5, 1.5, D).astype(np.float32)
        beta = rng.uniform(-1, 1, D).astype(np.float32)
        y, s = orc.layer_norm(x, gamma, beta, 1e-5, add=add, want_sum=True)
        assert (s == x + add).all()
        xs = s.astype(np.float64)
        c = xs - xs.mean(1, keepdims=True)
        ref = c / np.sqrt((c * c).mean(1, keepdims=True) + np.float64(np.float32(1e-5))) * gamma + beta
        assert np.abs(y - ref).max() <= 2e-6 * np.abs(ref).max()


def test_layer_norm_constant_row_is_beta(orc):
    D = 64
    x = np.full((1, D), -2.5, np.float32)
    beta = np.linspace(0, 1, D).astype(np.float32)
    assert (orc.layer_norm(x, np.ones(D, np.float32), beta) == beta).all()


@pytest.mark.parametrize("causal", [True, False])
def test_sdpa_matches_float64(orc, causal):
    rng = np.random.default_rng(1)
    B, H, S, D = 2, 3, 70, 64
    q, k, v = (rng.standard_normal((B * S, H * D)).astype(np.float32) for _ in range(3))
    got = orc.sdpa(q, k, v, B, H, S, D, 0.125, causal)
    ref = np.zeros((B * S, H * D))
    for b in range(B):
        for h in range(H):
            sl, hs = slice(b * S, (b + 1) * S), slice(h * D, (h + 1) * D)
            sc = q[sl, hs].astype(np.float64) @ k[sl, hs].astype(np.float64).T * 0.125
            if causal:
                sc[np.triu_indices(S, 1)] = -np.inf
            w = np.exp(sc - sc.max(1, keepdims=True))
            ref[sl, hs] = (w / w.sum(1, keepdims=True)) @ v[sl, hs].astype(np.float64)
    assert np.abs(got - ref).max() <= 2e-6 * np.abs(ref).max()
    rows = np.array([0, 69, 70, (1 * H + 2) * S + 33])
    part = orc.sdpa(q, k, v, B, H, S, D, 0.125, causal, rows=rows)
    for t, f in enumerate(rows):
        i, bh = f % S, f // S
        assert (part[t] == got[(bh // H) * S + i, (bh % H) * D:(bh % H + 1) * D]).all()


def test_first_causal_row_is_its_value(orc):
    rng = np.random.default_rng(2)
    q, k, v = (rng.standard_normal((8, 64)).astype(np.float32) for _ in range(3))
    out = orc.sdpa(q, k, v, 1, 1, 8, 64, 0.125, True)
    assert (out[0] == v[0]).all()
