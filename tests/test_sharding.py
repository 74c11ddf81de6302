"""Multi-rank host logic on CPU: row / column block arithmetic, and the column-sharded stack run by two gloo ranks
with a CPU stand-in for the device computation (the oracle), compared with the unsharded chain."""
import os
import socket

import numpy as np
import pytest

from mlfw_b200.sharding import (ColumnShardedStack, ShardedLayer, chunk_rows, column_block, from_gathered_layout, gather_columns,
                                gather_layout, range_from_keys, range_keys, row_block, to_gathered_layout)


def test_row_blocks_partition_the_rows():
    for M in (0, 1, 7, 8, 8192, 8191):
        for world in (1, 2, 4, 8):
            blocks = [row_block(M, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and sum(c for _, c in blocks) == M
            assert all(blocks[i][0] + blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            assert max(c for _, c in blocks) - min(c for _, c in blocks) <= 1


def test_column_blocks_are_tile_aligned_and_cover_n():
    for N in (256, 768, 3072, 8192, 28672, 1000, 100):
        for world in (1, 2, 4, 8):
            blocks = gather_layout(N, world)
            assert blocks[0][0] == 0 and sum(c for _, c in blocks) == N
            pos = 0
            for start, cols in blocks:
                assert start == pos or cols == 0
                assert start % 256 == 0 or cols == 0
                pos += cols
    assert gather_layout(28672, 8) == [(i * 3584, 3584) for i in range(8)]
    assert gather_layout(8192, 8) == [(i * 1024, 1024) for i in range(8)]


def test_range_keys_order_like_the_values_and_round_trip():
    vals = np.array([-np.inf, -3e38, -1.5, -1e-45, -0.0, 0.0, 1e-45, 2.5, 3e38, np.inf], np.float32)
    keys = range_keys(vals, vals)
    kmax, kmin = keys[:vals.size].astype(np.int64), keys[vals.size:].astype(np.int64)
    assert kmax[0] == 0 and (np.diff(kmax[1:]) > 0).all() and (kmax[1:] > 0).all()       # -inf as a maximum = nothing seen
    assert kmin[-1] == 0 and (np.diff(kmin[:-1]) < 0).all() and (kmin[:-1] > 0).all()    # +inf as a minimum = nothing seen
    mn, mx = range_from_keys(keys)
    assert (mx[1:].view(np.uint32) == vals[1:].view(np.uint32)).all() and mx[0] == -np.inf
    assert (mn[:-1].view(np.uint32) == vals[:-1].view(np.uint32)).all() and mn[-1] == np.inf
    nan = np.array([np.nan], np.float32)
    assert (range_keys(nan, nan) == 0).all()
    # the maximum of two ranks' keys is the key of the joint range
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((2, 100)).astype(np.float32) * 50, rng.standard_normal((2, 100)).astype(np.float32) * 50
    lo1, hi1, lo2, hi2 = np.minimum(a[0], a[1]), np.maximum(a[0], a[1]), np.minimum(b[0], b[1]), np.maximum(b[0], b[1])
    mn, mx = range_from_keys(np.maximum(range_keys(lo1, hi1), range_keys(lo2, hi2)))
    assert (mn == np.minimum(lo1, lo2)).all() and (mx == np.maximum(hi1, hi2)).all()


def test_gathered_layout_round_trip_and_chunks():
    assert [chunk_rows(4096, 4, c) for c in range(4)] == [(0, 1024), (1024, 1024), (2048, 1024), (3072, 1024)]
    assert [chunk_rows(600, 2, c) for c in range(2)] == [(0, 512), (512, 88)]
    assert [chunk_rows(100, 3, c) for c in range(3)] == [(0, 100), (100, 0), (100, 0)]
    rng = np.random.default_rng(1)
    for M, N, world, chunks in [(600, 512, 4, 2), (700, 1024, 8, 3), (64, 256, 2, 1), (300, 384, 1, 2)]:
        a = rng.integers(-127, 128, size=(M, N)).astype(np.int8)
        g = to_gathered_layout(a, world, chunks)
        assert (from_gathered_layout(g, M, N, world, chunks) == a).all()
        if chunks == 1:      # one chunk: exactly what an all-gather of the ranks' [M, N/world] blocks produces
            cols = N // world
            assert (g.reshape(world, M, cols)[world - 1] == a[:, (world - 1) * cols:]).all()


class OracleOps:
    """CPU stand-in for the device computation (test infrastructure): numpy + the oracle, torch CPU tensors for the collectives."""

    def __init__(self, orc, torch):
        self.orc, self.torch = orc, torch

    def linear(self, q, scales, layer, M):
        acc = self.orc.qdot_i32(q.numpy(), layer.w)
        return self.torch.from_numpy(self.orc.epilogue(acc, scales.numpy(), layer.w_scales, layer.bias, layer.act))

    def row_range(self, y, M, cols):
        a = y.numpy()
        return self.torch.from_numpy(np.fmin.reduce(a, axis=1).astype(np.float32)), self.torch.from_numpy(np.fmax.reduce(a, axis=1).astype(np.float32))

    def to_keys(self, mn, mx):
        return self.torch.from_numpy(range_keys(mn.numpy(), mx.numpy()).astype(np.int64))     # gloo reduces int64

    def all_reduce_max(self, keys, dist):
        dist.all_reduce(keys, op=dist.ReduceOp.MAX)

    def from_keys(self, keys):
        mn, mx = range_from_keys(keys.numpy().astype(np.uint32))
        return self.torch.from_numpy(mn), self.torch.from_numpy(mx)

    def quantize_with_range(self, y, M, cols, mn, mx):
        # codes of each local element given the row's agreed range: append the two range ends to the row, quantize, drop them
        a = np.concatenate([y.numpy(), mn.numpy()[:, None], mx.numpy()[:, None]], axis=1)
        q, _, s = self.orc.quantize_per_token(a)
        return self.torch.from_numpy(np.ascontiguousarray(q[:, :cols])), self.torch.from_numpy(s)

    def all_gather_columns(self, local, M, layer, dist, world, dtype):
        return gather_columns(self.torch, dist, local, M, layer.N, world) if world > 1 else local


def full_case():
    rng = np.random.default_rng(11)
    M, dims = 24, [64, 768, 520, 64]              # 520: ragged, the last rank gets fewer columns
    x = rng.standard_normal((M, dims[0])).astype(np.float32)
    layers = []
    for i in range(3):
        K, N = dims[i], dims[i + 1]
        layers.append((rng.integers(-127, 128, size=(N, K)).astype(np.int8),
                       (rng.uniform(1e-3, 1e-2, N) / np.sqrt(K) * 8).astype(np.float32),
                       (rng.standard_normal(N) * 0.01).astype(np.float32), "silu" if i < 2 else "none"))
    return M, x, layers


def unsharded(orc, M, x, layers):
    q, _, s = orc.quantize_per_token(x)
    for i, (w, ws, b, act) in enumerate(layers):
        y = orc.epilogue(orc.qdot_i32(q, w), s, ws, b, act)
        if i == len(layers) - 1:
            return y
        q, _, s = orc.quantize_per_token(y)


def _rank_main(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    import oracle as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, x, layers = full_case()
        shards = []
        for w, ws, b, act in layers:
            N, K = w.shape
            c0, cols = column_block(N, world, rank)
            shards.append(ShardedLayer(K, N, c0, cols, np.ascontiguousarray(w[c0:c0 + cols]), ws[c0:c0 + cols].copy(), b[c0:c0 + cols].copy(), act))
        q, _, s = orc.quantize_per_token(x)
        stack = ColumnShardedStack(OracleOps(orc, torch), dist, rank, world, shards)
        y, _ = stack.forward(torch.from_numpy(q), torch.from_numpy(s), M, last_f32=True)
        np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_column_sharded_stack_matches_unsharded_chain(orc, tmp_path, world):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    M, x, layers = full_case()
    ref = unsharded(orc, M, x, layers)
    for r in range(world):
        y = np.load(tmp_path / f"y{r}.npy")
        assert y.shape == ref.shape
        assert (y.view(np.uint32) == ref.view(np.uint32)).all(), f"rank {r} differs from the unsharded chain"
