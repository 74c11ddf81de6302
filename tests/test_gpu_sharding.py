"""Device side of the column-sharded path on one GPU: the two-step per-token quantize (local row range, then codes from
an agreed range) reproduces the one-step kernel, and a single-rank ColumnShardedStack over DeviceOps matches the oracle."""
import numpy as np
import pytest

from gpu_util import Guarded, activations

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import mlfw_b200
    c = mlfw_b200.Context(0)
    yield c
    c.check_status()
    c.close()


def test_two_step_quantize_over_column_blocks(ctx, orc):
    rng = np.random.default_rng(2)
    M, N = 37, 1000
    y = activations(rng, M, N)
    y[3] = 1.5
    y[5, 17] = np.nan
    rq, _, rs = orc.quantize_per_token(y)
    dy = ctx.to_device(y)
    blocks = [(0, 256), (256, 512), (768, 232)]
    mins, maxs = [], []
    for c0, cols in blocks:
        mn, mx = Guarded(ctx, (M,), np.float32), Guarded(ctx, (M,), np.float32)
        ctx.row_range(dy.ptr + 4 * c0, M, cols, N, mn.ptr, mx.ptr)
        ctx.sync()
        mins.append(mn.download()); maxs.append(mx.download())
    gmn, gmx = np.fmin.reduce(mins), np.fmax.reduce(maxs)               # what the all-reduces compute
    dmn, dmx = ctx.to_device(gmn), ctx.to_device(gmx)
    dq = Guarded(ctx, (M, N), np.int8)
    ds = Guarded(ctx, (M,), np.float32)
    for c0, cols in blocks:
        ctx.quantize_rows_with_range(dy.ptr + 4 * c0, M, cols, N, dmn, dmx, dq.ptr + c0, N, ds.ptr)
    ctx.sync()
    assert (dq.download() == rq).all() and (ds.download().view(np.uint32) == rs.view(np.uint32)).all()


def test_single_rank_stack_on_device(ctx, orc):
    import torch
    from mlfw_b200 import sharding
    rng = np.random.default_rng(4)
    M, dims = 130, [256, 768, 512]
    dev = torch.device("cuda", 0)
    x = rng.standard_normal((M, dims[0])).astype(np.float32)
    layers, ref_layers = [], []
    for i in range(2):
        K, N = dims[i], dims[i + 1]
        w = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
        ws = (rng.uniform(1e-3, 1e-2, N) / np.sqrt(K) * 8).astype(np.float32)
        act = "silu" if i == 0 else "none"
        ref_layers.append((w, ws, act))
        layers.append(sharding.ShardedLayer(K, N, 0, N, torch.from_numpy(w).to(dev), torch.from_numpy(ws).to(dev), None, act))
    q, _, s = orc.quantize_per_token(x)
    stack = sharding.ColumnShardedStack(sharding.DeviceOps(ctx, torch), None, 0, 1, layers)
    y, _ = stack.forward(torch.from_numpy(q).to(dev), torch.from_numpy(s).to(dev), M, last_f32=True)
    h = orc.epilogue(orc.qdot_i32(q, ref_layers[0][0]), s, ref_layers[0][1], None, "silu")
    hq, _, hs = orc.quantize_per_token(h)
    ref = orc.epilogue(orc.qdot_i32(hq, ref_layers[1][0]), hs, ref_layers[1][1], None, "none")
    assert (y.cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all()
