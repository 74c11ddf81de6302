"""Device side of the column-sharded path on one GPU: the two-step per-token quantize (local row range, then codes from
an agreed range) reproduces the one-step kernel.  The sharded layers themselves are in test_gpu_group.py."""
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
