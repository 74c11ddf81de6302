"""Seeded synthetic inputs with the generators the reference uses for its own data.

mulberry32 as in src/util/random.ts:5-14; normals by Box-Muller pairs as in
src/tensor/factory/creation_ops.ts:61-75 / src/nn/init.ts:40-53 (``u1 || 1e-10``,
the literal 6.283185307179586); uniform as in src/nn/init.ts:31-38.  Vectorised
with numpy; every tensor gets its own generator, seeded ``seed * 1000003 + index``.
"""
from __future__ import annotations

import numpy as np


def tensor_seed(seed: int, index: int) -> int:
    return (seed * 1000003 + index) & 0xFFFFFFFF


def mulberry32(seed: int, n: int, start: int = 0) -> np.ndarray:
    """Outputs ``start .. start+n-1`` of makeRng(seed) as float64 in [0, 1) (the state is a counter, so any
    window of the stream can be produced directly)."""
    m = np.uint64(0xFFFFFFFF)
    a = (np.uint64(seed & 0xFFFFFFFF) + np.uint64(0x6D2B79F5) * np.arange(start + 1, start + n + 1, dtype=np.uint64)) & m
    t = ((a ^ (a >> np.uint64(15))) * (np.uint64(1) | a)) & m
    t = ((t + (((t ^ (t >> np.uint64(7))) * (np.uint64(61) | t)) & m)) & m) ^ t
    return ((t ^ (t >> np.uint64(14))) & m).astype(np.float64) / 4294967296.0


def normal(seed: int, shape, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    pairs = (n + 1) // 2
    u = mulberry32(seed, 2 * pairs)
    u1 = u[0::2]
    u1 = np.where(u1 == 0.0, 1e-10, u1)
    r = np.sqrt(-2.0 * np.log(u1))
    theta = 6.283185307179586 * u[1::2]
    out = np.empty(2 * pairs, np.float64)
    out[0::2] = mean + std * r * np.cos(theta)
    out[1::2] = mean + std * r * np.sin(theta)
    return out[:n].astype(np.float32).reshape(shape)


def uniform(seed: int, shape, a: float = 0.0, b: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    return (a + mulberry32(seed, n) * (b - a)).astype(np.float32).reshape(shape)


def randint_i8(seed: int, shape, lo: int = -127, hi: int = 127, chunk: int = 1 << 24) -> np.ndarray:
    n = int(np.prod(shape))
    out = np.empty(n, np.int8)
    for s0 in range(0, n, chunk):          # in pieces: the 64-bit temporaries of a 235 M-element weight would not fit comfortably
        k = min(chunk, n - s0)
        out[s0:s0 + k] = (np.floor(mulberry32(seed, k, s0) * (hi - lo + 1)).astype(np.int64) + lo).astype(np.int8)
    return out.reshape(shape)


def with_outliers(x: np.ndarray, seed_mask: int, seed_values: int, p: float = 0.001, std: float = 20.0) -> np.ndarray:
    """Replaces a Bernoulli(p) subset (own stream) by N(0, std) values (own stream)."""
    mask = mulberry32(seed_mask, x.size).reshape(x.shape) < p
    vals = normal(seed_values, x.shape, 0.0, std)
    return np.where(mask, vals, x).astype(np.float32)
