"""Several GPUs behind the C ABI (b200q_group_*), the two-step per-token requantization the column-sharded call is
built on, activations stored as gathered column blocks, captured steps and the bounded-wait self test.

Everything with world = 1 runs on one GPU (NCCL with a single rank); the cases with two or more ranks drive the GPUs
of one process through b200q_group_create and are skipped where the machine has fewer.  The bar is the same as
everywhere: int8 codes and scales bit-exact against the CPU oracle, f32 results of these tails bit-identical."""
import numpy as np
import pytest

from gpu_util import Guarded, activations
from mlfw_b200.sharding import from_gathered_layout

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import mlfw_b200
    c = mlfw_b200.Context(0)
    yield c
    c.check_status()
    c.close()


def _layer(rng, N, K, bias=True):
    w = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    ws = (rng.uniform(1e-3, 1e-2, N) / np.sqrt(K) * 8).astype(np.float32)
    b = (rng.standard_normal(N) * 0.05).astype(np.float32) if bias else None
    return w, ws, b


# ------------------------------------------------------------------ two-step requantization (one GPU)
@pytest.mark.parametrize("M,N,K,act", [(130, 512, 256, "silu"), (257, 1100, 144, "gelu_sigmoid"), (64, 4100, 128, "none"),
                                         (1030, 260, 512, "relu"), (5, 7, 16, "none"), (300, 3072, 768, "gelu_sigmoid")])
def test_requant_token_two_step_equals_full_quantize(ctx, orc, M, N, K, act):
    """Ranges out of the GEMM epilogue + one-pass encode == the oracle's per-token quantize of the f32 result, ragged
    shapes included (N not a multiple of 4 takes the element-wise encode); the kept f32 result is the linear's."""
    rng = np.random.default_rng(M + 3 * N + 7 * K)
    x = activations(rng, M, K)
    W, ws, bias = _layer(rng, N, K)
    q, _, s32 = orc.quantize_per_token(x)
    y = orc.epilogue(orc.qdot_i32(q, W), s32, ws, bias, act)
    rq, _, rs = orc.quantize_per_token(y)
    dq, dW, ds, dws, db = ctx.to_device(q), ctx.to_device(W), ctx.to_device(s32), ctx.to_device(ws), ctx.to_device(bias)
    for variant in (0, 1):
        ctx.set_requant_variant(variant)
        try:
            doq, dos, dy = Guarded(ctx, (M, N), np.int8), Guarded(ctx, (M,), np.float32), Guarded(ctx, (M, N), np.float32)
            ctx.int8_linear_requant_token(dq, ds, dW, dws, db, act, M, N, K, doq.ptr, dos.ptr)
            ctx.sync()
            assert (dos.download().view(np.uint32) == rs.view(np.uint32)).all(), f"scales, variant {variant}"
            assert (doq.download() == rq).all(), f"codes, variant {variant}"
            doq2, dos2 = Guarded(ctx, (M, N), np.int8), Guarded(ctx, (M,), np.float32)
            ctx.int8_linear_f32_requant_token(dq, ds, dW, dws, db, act, M, N, K, dy.ptr, doq2.ptr, dos2.ptr)
            ctx.sync()
            assert (dy.download().view(np.uint32) == y.astype(np.float32).view(np.uint32)).all()
            assert (doq2.download() == rq).all() and (dos2.download().view(np.uint32) == rs.view(np.uint32)).all()
        finally:
            ctx.set_requant_variant(0)


def test_requant_token_rows_with_nan_inf_and_constant(ctx, orc):
    """Rows whose result is constant (bias only), contains +-Inf or NaN: the published ranges follow the same rules as
    the range pass (NaN ignored, non-finite ends replaced, equal ends widened)."""
    rng = np.random.default_rng(77)
    M, N, K = 96, 512, 128
    x = activations(rng, M, K)
    x[3] = 0.0                                          # zero codes -> the row is the bias vector
    W, ws, bias = _layer(rng, N, K)
    bias[:] = 0.25
    bias[5] = np.inf
    bias[9] = -np.inf
    bias[17] = np.nan
    q, _, s32 = orc.quantize_per_token(x)
    y = orc.epilogue(orc.qdot_i32(q, W), s32, ws, bias, "none")
    rq, _, rs = orc.quantize_per_token(y)
    dq, dW, ds, dws, db = ctx.to_device(q), ctx.to_device(W), ctx.to_device(s32), ctx.to_device(ws), ctx.to_device(bias)
    doq, dos = Guarded(ctx, (M, N), np.int8), Guarded(ctx, (M,), np.float32)
    ctx.int8_linear_requant_token(dq, ds, dW, dws, db, "none", M, N, K, doq.ptr, dos.ptr)
    ctx.sync()
    assert (dos.download().view(np.uint32) == rs.view(np.uint32)).all()
    assert (doq.download() == rq).all()
    # all columns equal (constant rows): bias the same everywhere, zero activations
    bias[:] = -1.75
    db = ctx.to_device(bias)
    y = orc.epilogue(orc.qdot_i32(q, W), s32, ws, bias, "none")
    rq, _, rs = orc.quantize_per_token(y)
    ctx.int8_linear_requant_token(dq, ds, dW, dws, db, "none", M, N, K, doq.ptr, dos.ptr)
    ctx.sync()
    assert (dos.download().view(np.uint32) == rs.view(np.uint32)).all()
    assert (doq.download() == rq).all()


# ------------------------------------------------------------------ activations as gathered column blocks (one GPU)
@pytest.mark.parametrize("M,N,K,blocks", [(256, 512, 1024, 2), (130, 260, 1024, 8), (1100, 300, 512, 4), (64, 256, 384, 3)])
def test_linear_reads_gathered_column_blocks(ctx, orc, M, N, K, blocks):
    """The GEMM reads A laid out block after block ([blocks][M][K/blocks]) through a three-dimensional tensor map:
    same result as from the row-major matrix, for both tile forms (M below and from 1024 rows)."""
    rng = np.random.default_rng(M + K + blocks)
    A = rng.integers(-127, 128, size=(M, K)).astype(np.int8)
    s = rng.uniform(0.01, 0.05, M).astype(np.float32)
    W, ws, bias = _layer(rng, N, K)
    ref = orc.epilogue(orc.qdot_i32(A, W), s, ws, bias, "relu")
    pc = K // blocks
    gathered = np.ascontiguousarray(np.stack([A[:, r * pc:(r + 1) * pc] for r in range(blocks)], axis=0))
    dA, ds, dW, dws, db = ctx.to_device(gathered), ctx.to_device(s), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    out = Guarded(ctx, (M, N), np.float32)
    ctx.int8_linear_gathered(dA, ds, blocks, dW, dws, db, "relu", M, N, K, out.ptr)
    ctx.sync()
    assert (out.download().view(np.uint32) == ref.astype(np.float32).view(np.uint32)).all()


def test_gathered_blocks_must_be_multiples_of_128(ctx):
    import mlfw_b200
    d = ctx.empty((1024,), np.int8)
    with pytest.raises(mlfw_b200.B200QError, match="multiple of 128"):
        ctx.int8_linear_gathered(d, d, 2, d, d, None, "none", 4, 8, 192, d)


# ------------------------------------------------------------------ groups
def _stack_reference(orc, x, layers):
    """Unsharded chain on the CPU oracle: codes + scales after every requantized layer, f32 result of the last."""
    q, _, s = orc.quantize_per_token(x)
    stages = []
    for i, (w, ws, b, act) in enumerate(layers):
        y = orc.epilogue(orc.qdot_i32(q, w), s, ws, b, act)
        if i == len(layers) - 1:
            return stages, y.astype(np.float32), None
        q, _, s = orc.quantize_per_token(y)
        stages.append((q, s))


def _run_nshard_stack(orc, devices, M, dims, chunks, seed):
    import mlfw_b200
    rng = np.random.default_rng(seed)
    world = len(devices)
    x = activations(rng, M, dims[0])
    acts = ["silu"] * (len(dims) - 2) + ["none"]
    layers = []
    for i in range(len(dims) - 1):
        w, ws, b = _layer(rng, dims[i + 1], dims[i], bias=(i % 2 == 0))
        layers.append((w, ws, b, acts[i]))
    stages, ref_last, _ = _stack_reference(orc, x, layers)
    q0, _, s0 = orc.quantize_per_token(x)
    with mlfw_b200.Group(devices) as g:
        assert g.world == world and g.local_count == world and g.nccl_version() > 20000
        g.set_chunks(chunks)
        cs = g.contexts
        q_in = [c.to_device(q0) for c in cs]
        s_in = [c.to_device(s0) for c in cs]
        held = []
        in_blocks = 1
        for i, (w, ws, b, act) in enumerate(layers):
            K, N = dims[i], dims[i + 1]
            cols = N // world
            Wd = [c.to_device(np.ascontiguousarray(w[r * cols:(r + 1) * cols])) for r, c in enumerate(cs)]
            wsd = [c.to_device(ws[r * cols:(r + 1) * cols].copy()) for r, c in enumerate(cs)]
            bd = [c.to_device(b[r * cols:(r + 1) * cols].copy()) for r, c in enumerate(cs)] if b is not None else None
            held.append((Wd, wsd, bd, q_in, s_in))
            if i == len(layers) - 1:
                outs = [Guarded(c, (M, cols), np.float32) for c in cs]
                g.linear_nshard(q_in, s_in, in_blocks, Wd, wsd, bd, act, M, N, K, out_f32=[o.ptr for o in outs])
                g.sync()
                for r, o in enumerate(outs):
                    got = o.download()
                    assert (got.view(np.uint32) == ref_last[:, r * cols:(r + 1) * cols].copy().view(np.uint32)).all(), f"f32, rank {r}"
            else:
                q_out = [Guarded(c, (M, N), np.int8) for c in cs]
                s_out = [Guarded(c, (M,), np.float32) for c in cs]
                g.linear_nshard(q_in, s_in, in_blocks, Wd, wsd, bd, act, M, N, K, q_out=[o.ptr for o in q_out],
                                out_scales=[o.ptr for o in s_out])
                g.sync()
                rq, rs = stages[i]
                for r in range(world):
                    assert (s_out[r].download().view(np.uint32) == rs.view(np.uint32)).all(), f"scales, layer {i}, rank {r}"
                    assert (from_gathered_layout(q_out[r].download(), M, N, world, chunks) == rq).all(), f"codes, layer {i}, rank {r}"
                q_in, s_in = [o.ptr for o in q_out], [o.ptr for o in s_out]
                held.append((q_out, s_out))
                in_blocks = world
        for c in cs:
            c.check_status()


@pytest.mark.parametrize("chunks", [1, 2])
def test_group_of_one_rank_runs_the_column_sharded_stack(orc, chunks):
    _run_nshard_stack(orc, [0], 600, [256, 768, 512, 384], chunks, seed=5)


@pytest.mark.parametrize("world,chunks", [(2, 1), (2, 3), (4, 2), (8, 1)])
def test_column_sharded_stack_equals_unsharded(orc, world, chunks):
    """N-sharded layers over `world` GPUs of this process: codes, scales and the final f32 columns are bit for bit
    what one GPU computes (keys max-reduced and int8 blocks all-gathered by NCCL inside the library)."""
    import mlfw_b200
    if mlfw_b200._lib.lib().b200q_device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    _run_nshard_stack(orc, list(range(world)), 700, [512, 1024 * world // 2 if world > 2 else 1024, 1024, 256 * world], chunks,
                      seed=40 + world)


def test_row_sharded_group_equals_one_gpu(orc):
    import mlfw_b200
    n = min(mlfw_b200._lib.lib().b200q_device_count(), 4)
    rng = np.random.default_rng(9)
    M, N, K = 530, 512, 1024
    x = activations(rng, M, K)
    W, ws, bias = _layer(rng, N, K)
    ref, _, _, _ = orc.linear(x, W, ws, bias, "gelu_sigmoid")
    from mlfw_b200.sharding import row_block
    with mlfw_b200.Group(list(range(n))) as g:
        cs = g.contexts
        blocks = [row_block(M, n, r) for r in range(n)]
        xd = [c.to_device(x[r0:r0 + rows]) for c, (r0, rows) in zip(cs, blocks)]
        Wd, wsd, bd = [c.to_device(W) for c in cs], [c.to_device(ws) for c in cs], [c.to_device(bias) for c in cs]
        outs = [Guarded(c, (rows, N), np.float32) for c, (_, rows) in zip(cs, blocks)]
        g.linear_mshard(xd, [rows for _, rows in blocks], Wd, wsd, bd, "gelu_sigmoid", N, K, [o.ptr for o in outs])
        g.sync()
        got = np.concatenate([o.download() for o in outs], axis=0)
    assert (got.view(np.uint32) == ref.astype(np.float32).view(np.uint32)).all()


def test_group_all_gather_bytes(orc):
    import mlfw_b200
    n = min(mlfw_b200._lib.lib().b200q_device_count(), 4)
    with mlfw_b200.Group(list(range(n))) as g:
        cs = g.contexts
        pieces = [np.full(1000, 10 + r, np.uint8) for r in range(n)]
        send = [c.to_device(p) for c, p in zip(cs, pieces)]
        recv = [c.empty((n * 1000,), np.uint8) for c in cs]
        g.all_gather(send, recv, 1000)
        g.sync()
        for r in recv:
            assert (r.download() == np.concatenate(pieces)).all()


def test_column_sharded_call_rejects_bad_splits():
    import mlfw_b200
    with mlfw_b200.Group([0]) as g:
        c = g.contexts[0]
        d = c.empty((4096,), np.int8)
        with pytest.raises(mlfw_b200.B200QError, match="either q_out"):
            g.linear_nshard([d], [d], 1, [d], [d], None, "none", 4, 16, 16)
        with pytest.raises(mlfw_b200.B200QError, match="row-major"):
            g.linear_nshard([d], [d], 3, [d], [d], None, "none", 4, 16, 16, out_f32=[d])


# ------------------------------------------------------------------ captured steps
def test_captured_step_replays_bit_identically(ctx, orc):
    rng = np.random.default_rng(31)
    M, N, K = 1100, 512, 1024
    x = activations(rng, M, K)
    W, ws, bias = _layer(rng, N, K)
    ref, _, _, _ = orc.linear(x, W, ws, bias, "relu")
    dx, dW, dws, db = ctx.to_device(x), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    out = Guarded(ctx, (M, N), np.float32)
    ctx.linear_f32(dx, dW, dws, db, "relu", M, N, K, out.ptr)     # sizes every workspace
    ctx.sync()
    n0 = ctx.launch_count()
    ctx.graph_begin()
    ctx.linear_f32(dx, dW, dws, db, "relu", M, N, K, out.ptr)
    graph = ctx.graph_end()
    assert ctx.launch_count() == n0                               # nothing ran while recording
    try:
        for _ in range(3):
            out.raw.fill_bytes(0xA5)
            ctx.graph_launch(graph)
            ctx.sync()
            assert (out.download().view(np.uint32) == ref.astype(np.float32).view(np.uint32)).all()
        assert ctx.launch_count() == n0 + 3 * 2                   # quantize + GEMM per replay
    finally:
        ctx.graph_destroy(graph)


def test_recording_refuses_what_cannot_be_recorded(ctx):
    import mlfw_b200
    d = ctx.empty((16,), np.float32)
    ctx.graph_begin()
    try:
        with pytest.raises(mlfw_b200.B200QError, match="not allowed between"):
            ctx.sync()
        with pytest.raises(mlfw_b200.B200QError, match="not allowed between"):
            d.download()
    finally:
        graph = ctx.graph_end()
        ctx.graph_destroy(graph)


# ------------------------------------------------------------------ bounded wait
def test_bounded_wait_gives_up_and_reports(ctx):
    """A wait on a barrier nothing signals (one thread, nothing asynchronous in flight) runs out after its limit: the
    kernel returns, the status word carries the bit, clearing it works, and the context stays usable."""
    import time
    ctx.sync()
    assert ctx.status_word() == 0
    t0 = time.perf_counter()
    ctx.selftest_bounded_wait(0.02)
    ctx.sync()
    dt = time.perf_counter() - t0
    assert ctx.status_word() == 64
    assert 0.015 <= dt < 1.0, f"the wait took {dt:.3f} s for a 0.02 s limit"
    ctx.clear_status()
    assert ctx.status_word() == 0
    ctx.set_wait_limit(0.5)          # the setter used by the tensor-core kernel's waits
    ctx.set_wait_limit(2.0)
    x = np.arange(64 * 128, dtype=np.float32).reshape(64, 128)
    dq, ds = ctx.empty((64, 128), np.int8), ctx.empty((64,), np.float32)
    ctx.quantize_per_token(ctx.to_device(x), 64, 128, dq, ds)
    ctx.sync()
    ctx.check_status()
