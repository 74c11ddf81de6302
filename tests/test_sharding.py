"""Multi-rank host logic on CPU: row / column block arithmetic, and the column-sharded stack run by two gloo ranks
with a CPU stand-in for the device computation (the oracle), compared with the unsharded chain."""
import os
import socket

import numpy as np
import pytest

from mlfw_b200.sharding import ColumnShardedStack, ShardedLayer, column_block, gather_columns, gather_layout, row_block


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


class OracleOps:
    """CPU stand-in for DeviceOps (test infrastructure): numpy + the oracle, torch CPU tensors for the collectives."""

    def __init__(self, orc, torch):
        self.orc, self.torch = orc, torch

    def linear(self, q, scales, layer, M):
        acc = self.orc.qdot_i32(q.numpy(), layer.w)
        return self.torch.from_numpy(self.orc.epilogue(acc, scales.numpy(), layer.w_scales, layer.bias, layer.act))

    def row_range(self, y, M, cols):
        a = y.numpy()
        return self.torch.from_numpy(np.fmin.reduce(a, axis=1).astype(np.float32)), self.torch.from_numpy(np.fmax.reduce(a, axis=1).astype(np.float32))

    def all_reduce(self, v, op, dist):
        dist.all_reduce(v, op=dist.ReduceOp.MIN if op == "min" else dist.ReduceOp.MAX)

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
