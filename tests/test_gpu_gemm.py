"""GPU parity of the int8 contraction and its fused tail against the CPU oracle (through the C ABI).

int32 accumulators and int8 codes must be bit-exact.  f32 outputs of the relu / none /
sigmoid-GELU / SiLU tails are expected bit-exact as well (the device follows the same
rounding chain); the stated bar is 1e-5 of the output absmax, which is what gelu_tanh
(no reference counterpart) is held to.
"""
import numpy as np
import pytest

from gpu_util import Guarded, activations, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def ctx():
    import mlfw_b200
    c = mlfw_b200.Context(0)
    yield c
    c.check_status()
    c.close()


def gemm_inputs(rng, M, N, K):
    A = rng.integers(-127, 128, size=(M, K)).astype(np.int8)
    W = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    return A, W


# (M, N, K): ragged around the 64-wide tiles of the CUDA-core kernel and the 128x256x128 tiles of the tensor-core kernel
SIMT_SHAPES = [(1, 1, 1), (4, 6, 8), (64, 32, 128), (3, 5, 7), (65, 130, 67), (128, 256, 100), (200, 70, 333)]
UMMA_SHAPES = [(128, 256, 128), (1, 8, 16), (4, 6, 16), (64, 32, 128), (130, 260, 144), (256, 512, 1024), (128, 256, 4096),
               (300, 768, 768), (129, 257, 272), (512, 1024, 512), (127, 255, 112), (1024, 256, 2048)]


@pytest.mark.parametrize("M,N,K", SIMT_SHAPES + UMMA_SHAPES)
def test_gemm_i32_cuda_cores(ctx, orc, M, N, K):
    rng = np.random.default_rng(M * 1009 + N * 31 + K)
    A, W = gemm_inputs(rng, M, N, K)
    ctx.set_gemm_variant(1)
    try:
        dA, dW = Guarded(ctx, A.shape, np.int8, A), Guarded(ctx, W.shape, np.int8, W)
        dC = Guarded(ctx, (M, N), np.int32)
        ctx.int8_gemm_i32(dA.ptr, dW.ptr, M, N, K, dC.ptr)
        ctx.sync()
        assert (dC.download() == orc.qdot_i32(A, W)).all()
    finally:
        ctx.set_gemm_variant(0)


@pytest.mark.parametrize("zpA,zpW", [(3, 0), (0, -5), (-128, 127), (7, 9)])
def test_gemm_i32_zero_points(ctx, orc, zpA, zpW):
    rng = np.random.default_rng(3)
    M, N, K = 37, 45, 150
    A = rng.integers(-128, 128, size=(M, K)).astype(np.int8)
    W = rng.integers(-128, 128, size=(N, K)).astype(np.int8)
    dA, dW = Guarded(ctx, A.shape, np.int8, A), Guarded(ctx, W.shape, np.int8, W)
    dC = Guarded(ctx, (M, N), np.int32)
    ctx.int8_gemm_i32(dA.ptr, dW.ptr, M, N, K, dC.ptr, zpA, zpW)
    ctx.sync()
    assert (dC.download() == orc.qdot_i32(A, W, "NK", zpA, zpW)).all()


# gemm variants: 1 = CUDA cores, 2 = tensor cores with one CTA per 128x256 tile, 3 = CTA pairs on 256x256 tiles
@pytest.mark.parametrize("variant", [2, 3])
@pytest.mark.parametrize("M,N,K", UMMA_SHAPES + [(2048, 512, 256), (1300, 300, 160)])
def test_gemm_i32_tensor_cores(ctx, orc, M, N, K, variant):
    rng = np.random.default_rng(M * 1009 + N * 31 + K + 1)
    A, W = gemm_inputs(rng, M, N, K)
    dA, dW = ctx.to_device(A), ctx.to_device(W)      # cudaMalloc alignment: the TMA path is taken
    dC = Guarded(ctx, (M, N), np.int32)
    ctx.set_gemm_variant(variant)
    try:
        ctx.int8_gemm_i32(dA.ptr, dW.ptr, M, N, K, dC.ptr)
        ctx.sync()
    finally:
        ctx.set_gemm_variant(0)
    ctx.check_status()
    C = dC.download()
    ref = orc.qdot_i32(A, W)
    assert (C == ref).all(), f"{int((C != ref).sum())} of {C.size} accumulators differ"


def test_gemm_i32_extreme_values(ctx, orc):
    """All -128 x -128 over K = 4096 reaches 2^26: far above 2^24, still exact in int32."""
    M, N, K = 128, 256, 4096
    A = np.full((M, K), -128, np.int8)
    W = np.full((N, K), -128, np.int8)
    W[::2] = 127
    dA, dW = ctx.to_device(A), ctx.to_device(W)
    dC = Guarded(ctx, (M, N), np.int32)
    ctx.int8_gemm_i32(dA.ptr, dW.ptr, M, N, K, dC.ptr)
    ctx.sync()
    assert (dC.download() == orc.qdot_i32(A, W)).all()


def linear_case(rng, M, N, K, big_acc=False):
    x = activations(rng, M, K)
    W = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    ws = rng.uniform(1e-3, 1e-2, size=N).astype(np.float32) / np.float32(np.sqrt(K) / 8)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    if big_acc:
        W[: N // 2] = 127          # correlated weights and codes in [64,127]: accumulators beyond 2^24
        x = rng.uniform(0.5, 1.0, size=(M, K)).astype(np.float32)
    return x, W, ws, bias


ACTS = ["none", "relu", "gelu_sigmoid", "silu", "gelu_tanh"]
EXACT_ACTS = {"none", "relu", "gelu_sigmoid", "silu"}


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("M,N,K", [(256, 512, 1024), (130, 260, 144), (64, 1000, 768), (5, 7, 16), (136, 264, 4096)])
def test_int8_linear_fused_tail(ctx, orc, M, N, K, act, variant):
    rng = np.random.default_rng(M + N + K + len(act))
    x, W, ws, bias = linear_case(rng, M, N, K)
    q, _, s32 = orc.quantize_per_token(x)
    acc = orc.qdot_i32(q, W)
    ref = orc.epilogue(acc, s32, ws, bias, act)
    ctx.set_gemm_variant(variant)
    try:
        dq, dW = ctx.to_device(q), ctx.to_device(W)
        ds, dws, db = ctx.to_device(s32), ctx.to_device(ws), ctx.to_device(bias)
        dout = Guarded(ctx, (M, N), np.float32)
        ctx.int8_linear(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, act, M, N, K, dout.ptr)
        ctx.sync()
        ctx.check_status()
    finally:
        ctx.set_gemm_variant(0)
    out = dout.download()
    assert rel_err(out, ref) <= TOL
    if act in EXACT_ACTS:
        nd = int((out.view(np.uint32) != ref.view(np.uint32)).sum())
        assert nd == 0, f"{nd} of {out.size} f32 outputs are not bit-identical to the oracle"


def test_int8_linear_large_accumulators(ctx, orc):
    """|acc| >= 2^24: the int -> f32 conversion of the reference is NOT rounded before the multiply."""
    rng = np.random.default_rng(99)
    M, N, K = 128, 256, 4096
    x, W, ws, bias = linear_case(rng, M, N, K, big_acc=True)
    q, _, s32 = orc.quantize_per_token(x)
    acc = orc.qdot_i32(q, W)
    assert np.abs(acc).max() >= 2 ** 24
    ref = orc.epilogue(acc, s32, ws, bias, "none")
    dq, dW = ctx.to_device(q), ctx.to_device(W)
    ds, dws, db = ctx.to_device(s32), ctx.to_device(ws), ctx.to_device(bias)
    dout = Guarded(ctx, (M, N), np.float32)
    ctx.int8_linear(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, "none", M, N, K, dout.ptr)
    ctx.sync()
    assert (dout.download().view(np.uint32) == ref.view(np.uint32)).all()


def test_int8_linear_static_scale_no_bias(ctx, orc):
    """Reference scheme: static activation scale folded into sv[n] by the host (quantization_pass.ts:427-437)."""
    rng = np.random.default_rng(5)
    M, N, K = 64, 128, 256
    x = activations(rng, M, K, outliers=False)
    a_scale = 6 / 127
    q = orc.quantize_static(x, a_scale, 0)
    W = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    wsc = rng.uniform(1e-3, 1e-2, size=N)
    sv = (a_scale * wsc).astype(np.float32)
    ref = orc.epilogue_sv(orc.qdot_i32(q, W), sv, None, "relu")
    dx = ctx.to_device(x)
    dq = ctx.empty((M, K), np.int8)
    ctx.quantize_static(dx.ptr, M * K, a_scale, 0, 0, dq.ptr)
    dW, dsv = ctx.to_device(W), ctx.to_device(sv)
    dout = Guarded(ctx, (M, N), np.float32)
    ctx.int8_linear(dq.ptr, None, dW.ptr, dsv.ptr, None, "relu", M, N, K, dout.ptr)
    ctx.sync()
    assert (dq.download() == q).all()
    assert (dout.download().view(np.uint32) == ref.view(np.uint32)).all()


# N = 520: rows are not 16-byte multiples (lane-wise stores); 768: whole 64-code groups through the staging tile;
# 528 and 272: the last group of a row is partial and clipped by the bulk store.
@pytest.mark.parametrize("M,N,K", [(200, 520, 256), (300, 768, 256), (200, 528, 256), (1100, 272, 128)])
@pytest.mark.parametrize("variant", [1, 2, 3])
def test_int8_linear_requant_static(ctx, orc, variant, M, N, K):
    rng = np.random.default_rng(17 + N)
    x, W, ws, bias = linear_case(rng, M, N, K)
    q, _, s32 = orc.quantize_per_token(x)
    y = orc.epilogue(orc.qdot_i32(q, W), s32, ws, bias, "relu")
    out_scale = float(np.abs(y).max()) / 127
    ref = orc.quantize_static(y, out_scale, 0)
    ctx.set_gemm_variant(variant)
    try:
        dq, dW = ctx.to_device(q), ctx.to_device(W)
        ds, dws, db = ctx.to_device(s32), ctx.to_device(ws), ctx.to_device(bias)
        dout = Guarded(ctx, (M, N), np.int8)
        ctx.int8_linear_requant_static(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, "relu", M, N, K, out_scale, dout.ptr)
        ctx.sync()
    finally:
        ctx.set_gemm_variant(0)
    assert (dout.download() == ref).all()


def test_int8_linear_requant_token(ctx, orc):
    rng = np.random.default_rng(18)
    M, N, K = 130, 512, 256
    x, W, ws, bias = linear_case(rng, M, N, K)
    q, _, s32 = orc.quantize_per_token(x)
    y = orc.epilogue(orc.qdot_i32(q, W), s32, ws, bias, "silu")
    rq, _, rs = orc.quantize_per_token(y)
    dq, dW = ctx.to_device(q), ctx.to_device(W)
    ds, dws, db = ctx.to_device(s32), ctx.to_device(ws), ctx.to_device(bias)
    doq = Guarded(ctx, (M, N), np.int8)
    dos = Guarded(ctx, (M,), np.float32)
    ctx.int8_linear_requant_token(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, "silu", M, N, K, doq.ptr, dos.ptr)
    ctx.sync()
    assert (dos.download().view(np.uint32) == rs.view(np.uint32)).all()
    assert (doq.download() == rq).all()


@pytest.mark.parametrize("M,N,K", [(256, 1024, 512), (33, 100, 48), (7, 9, 10)])
def test_linear_f32_whole_path(ctx, orc, M, N, K):
    """f32 activations -> per-token quantize -> contraction -> tail, device and host-buffer entry points."""
    rng = np.random.default_rng(M * N + K)
    x, W, ws, bias = linear_case(rng, M, N, K)
    ref, _, _, _ = orc.linear(x, W, ws, bias, "relu")
    dx, dW, dws, db = ctx.to_device(x), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    dout = Guarded(ctx, (M, N), np.float32)
    ctx.linear_f32(dx.ptr, dW.ptr, dws.ptr, db.ptr, "relu", M, N, K, dout.ptr)
    ctx.sync()
    assert (dout.download().view(np.uint32) == ref.view(np.uint32)).all()
    out_host = np.zeros((M, N), np.float32)
    ctx.linear_f32_host(x, dW.ptr, dws.ptr, db.ptr, "relu", M, N, K, out_host)
    assert (out_host.view(np.uint32) == ref.view(np.uint32)).all()


@pytest.mark.parametrize("in_locked,out_locked", [(False, False), (True, False), (False, True), (True, True)])
def test_linear_f32_host_pipelines_row_blocks(ctx, in_locked, out_locked, M=5000, N=384, K=256):
    """Five row blocks through the host-buffer entry point: ordinary (pageable) arrays are staged through the context's
    page-locked ring by its copy threads, page-locked arrays go to the copy engines directly; every combination gives
    the device path's bits, twice in a row (the ring and its events are reused)."""
    rng = np.random.default_rng(77)
    x, W, ws, bias = linear_case(rng, M, N, K)
    dx, dW, dws, db = ctx.to_device(x), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    dout = ctx.empty((M, N), np.float32)
    ctx.linear_f32(dx, dW, dws, db, "gelu_sigmoid", M, N, K, dout)
    ctx.sync()
    ref = dout.download()
    hx = ctx.pinned((M, K), np.float32) if in_locked else None
    hy = ctx.pinned((M, N), np.float32) if out_locked else None
    xin = hx if in_locked else x.copy()
    if in_locked:
        hx.array[...] = x
    for _ in range(2):
        out = hy if out_locked else np.full((M, N), np.nan, np.float32)
        if out_locked:
            hy.array[...] = np.nan
        ctx.linear_f32_host(xin, dW.ptr, dws.ptr, db.ptr, "gelu_sigmoid", M, N, K, out)
        got = hy.array if out_locked else out
        assert (got.view(np.uint32) == ref.view(np.uint32)).all()
    for h in (hx, hy):
        if h is not None:
            h.free()


def test_linear_f32_host_with_arrays_registered_in_place(ctx, M=5000, N=384, K=256):
    """Ordinary numpy arrays page-locked in place (b200q_host_register) take the direct path of the host-buffer entry
    point and give the bits of the staged path; after unregistering they are ordinary arrays again."""
    rng = np.random.default_rng(78)
    x, W, ws, bias = linear_case(rng, M, N, K)
    dW, dws, db = ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    staged = np.full((M, N), np.nan, np.float32)
    ctx.linear_f32_host(x, dW.ptr, dws.ptr, db.ptr, "silu", M, N, K, staged)
    out = np.full((M, N), np.nan, np.float32)
    ctx.host_register(x)
    ctx.host_register(out)
    try:
        for _ in range(2):
            out[...] = np.nan
            ctx.linear_f32_host(x, dW.ptr, dws.ptr, db.ptr, "silu", M, N, K, out)
            assert (out.view(np.uint32) == staged.view(np.uint32)).all()
    finally:
        ctx.host_unregister(x)
        ctx.host_unregister(out)
    out[...] = np.nan
    ctx.linear_f32_host(x, dW.ptr, dws.ptr, db.ptr, "silu", M, N, K, out)
    assert (out.view(np.uint32) == staged.view(np.uint32)).all()
    import mlfw_b200
    with pytest.raises(mlfw_b200.B200QError):
        ctx.host_unregister(out)          # not registered any more


@pytest.mark.parametrize("count,M,N,K", [(1, 300, 256, 512), (2, 1100, 512, 256), (5, 2048, 768, 1024), (4, 70, 100, 48)])
def test_linear_f32_many_equals_batch_by_batch(ctx, count, M, N, K):
    """Independent batches with the quantize of the next one overlapping the GEMM of the current one (two streams, two
    sets of codes): every batch has the bits of b200q_linear_f32, also when the call is repeated and followed by a plain one."""
    rng = np.random.default_rng(count * 1000 + M)
    _, W, ws, bias = linear_case(rng, M, N, K)
    dW, dws, db = ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    xs = [activations(rng, M, K) for _ in range(count)]
    dxs = [ctx.to_device(x) for x in xs]
    refs = []
    dref = ctx.empty((M, N), np.float32)
    for dx in dxs:
        ctx.linear_f32(dx, dW, dws, db, "silu", M, N, K, dref)
        ctx.sync()
        refs.append(dref.download())
    outs = [Guarded(ctx, (M, N), np.float32) for _ in range(count)]
    for _ in range(2):
        ctx.linear_f32_many(dxs, dW, dws, db, "silu", M, N, K, [o.ptr for o in outs])
        ctx.linear_f32(dxs[0], dW, dws, db, "silu", M, N, K, dref)      # queued right behind: reuses the first set of codes
        ctx.sync()
        for o, r in zip(outs, refs):
            assert (o.download().view(np.uint32) == r.view(np.uint32)).all()
        assert (dref.download().view(np.uint32) == refs[0].view(np.uint32)).all()
    ctx.check_status()


@pytest.mark.parametrize("M,N,K,za,zw", [(256, 512, 1024, 5, -9), (1100, 384, 4096, -128, 127), (129, 70, 48, 3, 0), (64, 64, 16, 0, -7)])
def test_zero_points_on_the_tensor_cores(ctx, orc, M, N, K, za, zw):
    """sum (a - za)(w - zw) as the plain tensor-core product plus the three correction terms equals the CUDA-core
    kernel that subtracts tap by tap, and the oracle."""
    rng = np.random.default_rng(M + K)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    W = rng.integers(-128, 128, (N, K), dtype=np.int8)
    dA, dW = ctx.to_device(A), ctx.to_device(W)
    d0, d1 = Guarded(ctx, (M, N), np.int32), Guarded(ctx, (M, N), np.int32)
    ctx.set_gemm_variant(0)
    ctx.int8_gemm_i32(dA.ptr, dW.ptr, M, N, K, d0.ptr, za, zw)
    ctx.set_gemm_variant(1)
    ctx.int8_gemm_i32(dA.ptr, dW.ptr, M, N, K, d1.ptr, za, zw)
    ctx.set_gemm_variant(0)
    ctx.sync()
    got = d0.download()
    assert (got == d1.download()).all()
    assert (got == orc.qdot_i32(A, W, "NK", za, zw)).all()


@pytest.mark.parametrize("M,N,K", [(1300, 1100, 256), (2600, 520, 128), (256, 3000, 64)])
def test_tile_walking_order_does_not_change_results(ctx, orc, M, N, K):
    """The persistent CTAs may walk the tiles row block by row block or in groups of row blocks (groups that do not
    divide the row blocks, a group larger than the matrix): same accumulators, same f32 results, same row ranges."""
    rng = np.random.default_rng(M + N)
    x, W, ws, bias = linear_case(rng, M, N, K)
    q, _, s = orc.quantize_per_token(x)
    dq, dsc, dW, dws, db = ctx.to_device(q), ctx.to_device(s), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    ref_acc = orc.qdot_i32(q, W)
    results = []
    for g in (0, 1, 3, 8, 1000, -1):
        ctx.set_tile_group(g)
        dacc, dy = Guarded(ctx, (M, N), np.int32), Guarded(ctx, (M, N), np.float32)
        dqo, dso = Guarded(ctx, (M, N), np.int8), Guarded(ctx, (M,), np.float32)
        ctx.int8_gemm_i32(dq, dW, M, N, K, dacc.ptr)
        ctx.int8_linear_f32_requant_token(dq, dsc, dW, dws, db, "silu", M, N, K, dy.ptr, dqo.ptr, dso.ptr)
        ctx.sync()
        assert (dacc.download() == ref_acc).all()
        results.append((dy.download(), dqo.download(), dso.download()))
    ctx.set_tile_group(-1)
    for y, qo, so in results[1:]:
        assert (y.view(np.uint32) == results[0][0].view(np.uint32)).all() and (qo == results[0][1]).all()
        assert (so.view(np.uint32) == results[0][2].view(np.uint32)).all()
    ctx.check_status()


def test_epilogue_separate_op(ctx, orc):
    """convert -> mul(scale vector) -> add(bias) -> activation as its own kernel (the reference's unfused chain)."""
    rng = np.random.default_rng(23)
    M, N = 70, 130
    acc = rng.integers(-2 ** 27, 2 ** 27, size=(M, N)).astype(np.int32)
    a = rng.uniform(0.01, 0.05, M).astype(np.float32)
    w = rng.uniform(1e-5, 1e-4, N).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    for act in ["none", "relu", "gelu_sigmoid", "silu"]:
        ref = orc.epilogue(acc, a, w, b, act)
        dacc, da, dw, db = ctx.to_device(acc), ctx.to_device(a), ctx.to_device(w), ctx.to_device(b)
        dout = Guarded(ctx, (M, N), np.float32)
        ctx.epilogue(dacc.ptr, M, N, da.ptr, dw.ptr, db.ptr, act, dout.ptr)
        ctx.sync()
        assert (dout.download().view(np.uint32) == ref.view(np.uint32)).all(), act


def test_quant_roundtrip_host(ctx, orc):
    rng = np.random.default_rng(29)
    M, K = 64, 512
    x = activations(rng, M, K)
    q = np.zeros((M, K), np.int8)
    s = np.zeros(M, np.float32)
    y = np.zeros((M, K), np.float32)
    ctx.quant_roundtrip_host(x, M, K, q, s, y)
    rq, _, rs = orc.quantize_per_token(x)
    assert (q == rq).all() and (s == rs).all()
    assert (y == orc.dequantize_per_token_f32(rq, rs)).all()


@pytest.mark.parametrize("act", ["gelu_sigmoid", "silu", "relu", "gelu_tanh"])
def test_fused_tail_extreme_arguments(ctx, orc, act):
    """Pre-activations far outside the tame range (exp overflow side, NaN, +-Inf) take the general path."""
    rng = np.random.default_rng(41)
    M, N, K = 128, 256, 64
    x = activations(rng, M, K, outliers=False)
    W = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    ws = np.full(N, 1e-4, np.float32)
    specials = np.array([-200.0, -90.0, -87.5, -60.0, -51.5, -50.5, -30.0, 0.0, 30.0, 100.0, 1e30, -1e30, np.nan, np.inf,
                         -np.inf, 3.0], np.float32)
    bias = np.tile(specials, N // specials.size)
    q, _, s32 = orc.quantize_per_token(x)
    ref = orc.epilogue(orc.qdot_i32(q, W), s32, ws, bias, act)
    dq, dW = ctx.to_device(q), ctx.to_device(W)
    ds, dws, db = ctx.to_device(s32), ctx.to_device(ws), ctx.to_device(bias)
    dout = Guarded(ctx, (M, N), np.float32)
    ctx.int8_linear(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, act, M, N, K, dout.ptr)
    ctx.sync()
    out = dout.download()
    assert (np.isnan(out) == np.isnan(ref)).all()
    ok = ~np.isnan(ref)
    if act in EXACT_ACTS:
        assert (out[ok].view(np.uint32) == ref[ok].view(np.uint32)).all()
    else:
        fin = np.isfinite(ref)
        assert (out[ok & ~fin] == ref[ok & ~fin]).all()
        assert np.abs(out[fin].astype(np.float64) - ref[fin]).max() <= TOL * np.abs(ref[fin]).max()


@pytest.mark.parametrize("K", [64, 4096])
@pytest.mark.parametrize("act", ["gelu_sigmoid", "silu"])
def test_sigmoid_tail_argument_sweep(ctx, orc, act, K):
    """The exact sigmoid tails over their whole argument range: a dense sweep, runs of neighbouring floats around the
    overflow threshold of exp (88.72...), around the clamp where 1 + exp(x) rounds to 1 (-18) and around zero.  The
    accumulators are zero, so the pre-activation is the bias itself.  K 64 runs the binary64 form of the tail, K 4096
    the binary32 form (some of its arguments land on the binary64 redo)."""
    rng = np.random.default_rng(43)
    M, N = 128, 8192
    q = np.zeros((M, K), np.int8)
    s32 = np.ones(M, np.float32)
    W = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    ws = np.full(N, 1e-3, np.float32)
    k = 1.0 if act == "silu" else 1.0 / 1.702

    def run_of_neighbours(center, n):
        v = np.empty(n, np.float32)
        v[n // 2] = np.float32(center)
        for i in range(n // 2 + 1, n):
            v[i] = np.nextafter(v[i - 1], np.float32(np.inf))
        for i in range(n // 2 - 1, -1, -1):
            v[i] = np.nextafter(v[i + 1], np.float32(-np.inf))
        return v

    biases = [np.linspace(-91.0 * k, 21.0 * k, N).astype(np.float32),
              (rng.uniform(-90.0, 20.0, N) * k).astype(np.float32),
              np.concatenate([run_of_neighbours(-88.7228394 * k, 2048), run_of_neighbours(-88.75 * k, 1024),
                              run_of_neighbours(18.0 * k, 2048), run_of_neighbours(0.0, 1024),
                              run_of_neighbours(-1.0 / 256 * k, 1024), run_of_neighbours(17.32868 * k, 1024)])]
    dq, dW, ds, dws = ctx.to_device(q), ctx.to_device(W), ctx.to_device(s32), ctx.to_device(ws)
    for bias in biases:
        assert bias.size == N
        ref = orc.epilogue(np.zeros((M, N), np.int32), s32, ws, bias, act)
        db = ctx.to_device(bias)
        dout = Guarded(ctx, (M, N), np.float32)
        ctx.int8_linear(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, act, M, N, K, dout.ptr)
        ctx.sync()
        ctx.check_status()
        out = dout.download()
        nd = int((out.view(np.uint32) != ref.view(np.uint32)).sum())
        assert nd == 0, f"{nd} of {out.size} outputs differ from the oracle"


@pytest.mark.parametrize("act", ["gelu_sigmoid", "silu"])
@pytest.mark.parametrize("M,N,K", [(300, 768, 768), (1100, 512, 256)])
def test_approximate_tail_mode(ctx, orc, act, M, N, K):
    """Tail mode 1: hardware exp / reciprocal for f32 outputs -- inside the 1e-5 bar; int8 outputs stay exact."""
    rng = np.random.default_rng(M + N + K)
    x, W, ws, bias = linear_case(rng, M, N, K)
    ws = ws * 40          # pre-activations far into both saturated ends of the sigmoid
    q, _, s32 = orc.quantize_per_token(x)
    acc = orc.qdot_i32(q, W)
    ref = orc.epilogue(acc, s32, ws, bias, act)
    dq, dW = ctx.to_device(q), ctx.to_device(W)
    ds, dws, db = ctx.to_device(s32), ctx.to_device(ws), ctx.to_device(bias)
    dout = Guarded(ctx, (M, N), np.float32)
    dcodes = Guarded(ctx, (M, N), np.int8)
    out_scale = float(np.abs(ref).max()) / 127
    ctx.set_tail_mode(1)
    try:
        ctx.int8_linear(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, act, M, N, K, dout.ptr)
        ctx.int8_linear_requant_static(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, act, M, N, K, out_scale, dcodes.ptr)
        ctx.sync()
    finally:
        ctx.set_tail_mode(0)
    got = dout.download()
    assert rel_err(got, ref) <= TOL
    assert not (got.view(np.uint32) == ref.view(np.uint32)).all()          # it really is the other code path
    assert (dcodes.download() == orc.quantize_static(ref, out_scale, 0)).all()
    ctx.int8_linear(dq.ptr, ds.ptr, dW.ptr, dws.ptr, db.ptr, act, M, N, K, dout.ptr)   # back in mode 0: bit-exact again
    ctx.sync()
    assert (dout.download().view(np.uint32) == ref.view(np.uint32)).all()
