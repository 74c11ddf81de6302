"""GPU parity of the f32 pieces of a transformer block (embedding, LayerNorm + per-token quantize, attention, residual
add) against the CPU oracle, through the C ABI.

Copies and single additions are bit-exact.  LayerNorm and attention are floating-point reductions: within 1e-5 of the
output's largest magnitude (the tolerance the spec states).  The int8 codes and scales LayerNorm emits must be the
exact per-token quantization of the f32 values the same launch stored.
"""
import numpy as np
import pytest

from gpu_util import Guarded, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def ctx():
    import mlfw_b200
    c = mlfw_b200.Context(0)
    yield c
    c.check_status()
    c.close()


@pytest.mark.parametrize("M,D,V,S,pos", [(64, 768, 1000, 16, True), (33, 64, 50, 33, False), (1, 4, 3, 1, True), (512, 768, 50257, 128, True)])
def test_embedding(ctx, M, D, V, S, pos):
    rng = np.random.default_rng(M + D)
    table = rng.standard_normal((V, D)).astype(np.float32)
    ptab = rng.standard_normal((S, D)).astype(np.float32) if pos else None
    tokens = rng.integers(0, V, size=M).astype(np.int32)
    dt, dtok = ctx.to_device(table), ctx.to_device(tokens)
    dp = ctx.to_device(ptab) if pos else None
    out = Guarded(ctx, (M, D), np.float32)
    ctx.embedding_f32(dt, dtok, dp, M, D, V, S, out.ptr)
    ctx.sync()
    ref = table[tokens]
    if pos:
        ref = ref + ptab[np.arange(M) % S]
    assert (out.download().view(np.uint32) == ref.astype(np.float32).view(np.uint32)).all()


def test_embedding_bad_token_sets_status(ctx):
    table = np.ones((4, 8), np.float32)
    tokens = np.array([0, 7, -1, 3], np.int32)
    out = Guarded(ctx, (4, 8), np.float32)
    ctx.embedding_f32(ctx.to_device(table), ctx.to_device(tokens), None, 4, 8, 4, 0, out.ptr)
    ctx.sync()
    got = out.download()
    assert (got[[0, 3]] == 1).all() and (got[[1, 2]] == 0).all()
    assert ctx.status_word() & (1 << 5)
    ctx.clear_status()


@pytest.mark.parametrize("n", [4, 1000, 768 * 333])
def test_add(ctx, n):
    rng = np.random.default_rng(n)
    a, b = rng.standard_normal(n).astype(np.float32), (rng.standard_normal(n) * 100).astype(np.float32)
    out = Guarded(ctx, (n,), np.float32)
    ctx.add_f32(ctx.to_device(a), ctx.to_device(b), n, out.ptr)
    ctx.sync()
    assert (out.download().view(np.uint32) == (a + b).view(np.uint32)).all()


def run_layernorm(ctx, x, res, gamma, beta, eps, want=("sum", "y", "q")):
    M, D = x.shape
    dx = ctx.to_device(x)
    dr = ctx.to_device(res) if res is not None else None
    dg, db = ctx.to_device(gamma), ctx.to_device(beta)
    s = Guarded(ctx, (M, D), np.float32) if ("sum" in want and res is not None) else None
    y = Guarded(ctx, (M, D), np.float32) if "y" in want else None
    q = Guarded(ctx, (M, D), np.int8) if "q" in want else None
    sc = Guarded(ctx, (M,), np.float32) if "q" in want else None
    ctx.layernorm_quantize(dx, dr, dg, db, eps, M, D, s.ptr if s else None, y.ptr if y else None, q.ptr if q else None,
                           sc.ptr if sc else None)
    ctx.sync()
    return tuple(b.download() if b is not None else None for b in (s, y, q, sc))


@pytest.mark.parametrize("M,D", [(100, 768), (33, 64), (257, 1024), (64, 2048), (5, 36), (1, 4), (1000, 256), (19, 1536)])
@pytest.mark.parametrize("residual", [False, True])
def test_layernorm_quantize(ctx, orc, M, D, residual):
    rng = np.random.default_rng(M * 7 + D + residual)
    x = (rng.standard_normal((M, D)) * 3 + 0.5).astype(np.float32)
    res = rng.standard_normal((M, D)).astype(np.float32) if residual else None
    gamma = rng.uniform(0.5, 1.5, D).astype(np.float32)
    beta = rng.uniform(-0.5, 0.5, D).astype(np.float32)
    s, y, q, sc = run_layernorm(ctx, x, res, gamma, beta, 1e-5)
    ref_y, ref_s = orc.layer_norm(x, gamma, beta, 1e-5, add=res, want_sum=True)
    if residual:
        assert (s.view(np.uint32) == ref_s.view(np.uint32)).all()
    assert rel_err(y, ref_y) <= TOL
    # the codes are the exact per-token quantization of what the kernel stored as f32
    rq, _, rs = orc.quantize_per_token(y)
    assert (sc.view(np.uint32) == rs.view(np.uint32)).all()
    assert (q == rq).all()


def test_layernorm_codes_only_match_full_outputs(ctx, orc):
    rng = np.random.default_rng(5)
    M, D = 300, 768
    x = rng.standard_normal((M, D)).astype(np.float32)
    gamma, beta = np.ones(D, np.float32), np.zeros(D, np.float32)
    _, y, q, sc = run_layernorm(ctx, x, None, gamma, beta, 1e-5)
    _, _, q2, sc2 = run_layernorm(ctx, x, None, gamma, beta, 1e-5, want=("q",))
    assert (q == q2).all() and (sc.view(np.uint32) == sc2.view(np.uint32)).all()


def test_layernorm_edge_rows(ctx, orc):
    """A constant row (variance 0 -> beta everywhere), a row with a NaN, a row of large values."""
    D = 128
    x = np.zeros((4, D), np.float32)
    x[0] = 3.25
    x[1] = np.linspace(-1, 1, D)
    x[1, 7] = np.nan
    x[2] = np.linspace(-1, 1, D) * 1e18
    x[3] = np.linspace(-1, 1, D) * 1e-20
    gamma = np.full(D, 2.0, np.float32)
    beta = np.linspace(-1, 1, D).astype(np.float32)
    _, y, q, sc = run_layernorm(ctx, x, None, gamma, beta, 1e-5)
    ref = orc.layer_norm(x, gamma, beta, 1e-5)
    assert (y[0].view(np.uint32) == beta.view(np.uint32)).all()
    assert np.isnan(y[1]).all() and np.isnan(ref[1]).all()
    assert rel_err(y[2:], ref[2:]) <= TOL
    rq, _, rs = orc.quantize_per_token(y)
    assert (sc.view(np.uint32) == rs.view(np.uint32)).all()
    assert (q == rq).all()


def test_layernorm_nan_column(ctx, orc):
    """A NaN in beta poisons one column of every row; the other codes of those rows must not suffer."""
    rng = np.random.default_rng(12)
    M, D = 70, 768
    x = rng.standard_normal((M, D)).astype(np.float32)
    gamma = np.ones(D, np.float32)
    beta = np.zeros(D, np.float32)
    beta[100] = np.nan
    gamma[5] = np.inf
    _, y, q, sc = run_layernorm(ctx, x, None, gamma, beta, 1e-5)
    assert np.isnan(y[:, 100]).all()
    rq, _, rs = orc.quantize_per_token(y)
    assert (sc.view(np.uint32) == rs.view(np.uint32)).all()
    assert (q == rq).all()


def run_sdpa(ctx, q, k, v, B, H, S, scale, causal, packed=False):
    D = 64
    ld = H * D
    if packed:   # one [M, 3*H*64] buffer, as a fused q/k/v projection writes it
        qkv = np.concatenate([q, k, v], axis=1)
        dqkv = ctx.to_device(qkv)
        out = Guarded(ctx, (B * S, ld), np.float32)
        ctx.sdpa_f32(dqkv.ptr, dqkv.ptr + ld * 4, dqkv.ptr + 2 * ld * 4, 3 * ld, 3 * ld, 3 * ld, B, H, S, D, scale, causal, out.ptr, ld)
    else:
        out = Guarded(ctx, (B * S, ld), np.float32)
        ctx.sdpa_f32(ctx.to_device(q), ctx.to_device(k), ctx.to_device(v), ld, ld, ld, B, H, S, D, scale, causal, out.ptr, ld)
    ctx.sync()
    return out.download()


@pytest.mark.parametrize("B,H,S", [(2, 3, 70), (1, 2, 512), (3, 1, 1), (1, 1, 64), (2, 2, 65), (1, 12, 200)])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("variant", [0, 1, 3])   # tcgen05 / mma.sync (both with three-way tf32 products) / CUDA-core FMA
def test_sdpa(ctx, orc, B, H, S, causal, variant):
    rng = np.random.default_rng(B * 100 + H * 10 + S + causal)
    shape = (B * S, H * 64)
    q, k, v = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
    q *= 2.0   # sharper softmax rows
    ctx.set_sdpa_variant(variant)
    try:
        got = run_sdpa(ctx, q, k, v, B, H, S, 0.125, causal)
    finally:
        ctx.set_sdpa_variant(0)
    ref = orc.sdpa(q, k, v, B, H, S, 64, 0.125, causal)
    assert rel_err(got, ref) <= TOL


def test_sdpa_large_magnitudes(ctx, orc):
    """Scores far apart (one key dominates) and values of very different sizes: the split products must not lose them."""
    rng = np.random.default_rng(77)
    B, H, S = 1, 2, 192
    shape = (B * S, H * 64)
    q = (rng.standard_normal(shape) * 6).astype(np.float32)
    k = (rng.standard_normal(shape) * 6).astype(np.float32)
    v = (rng.standard_normal(shape) * np.exp(rng.uniform(-6, 6, size=shape))).astype(np.float32)
    for variant in (0, 1, 3):
        ctx.set_sdpa_variant(variant)
        try:
            got = run_sdpa(ctx, q, k, v, B, H, S, 0.125, True)
        finally:
            ctx.set_sdpa_variant(0)
        assert rel_err(got, orc.sdpa(q, k, v, B, H, S, 64, 0.125, True)) <= TOL


def test_sdpa_reads_packed_projections(ctx, orc):
    rng = np.random.default_rng(9)
    B, H, S = 2, 4, 130
    shape = (B * S, H * 64)
    q, k, v = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
    got = run_sdpa(ctx, q, k, v, B, H, S, 0.125, True, packed=True)
    assert rel_err(got, orc.sdpa(q, k, v, B, H, S, 64, 0.125, True)) <= TOL


def test_sdpa_causality(ctx):
    """Changing keys and values after position p leaves the outputs up to p untouched, bit for bit."""
    rng = np.random.default_rng(10)
    B, H, S, p = 1, 2, 200, 77
    shape = (B * S, H * 64)
    q, k, v = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
    a = run_sdpa(ctx, q, k, v, B, H, S, 0.125, True)
    k2, v2 = k.copy(), v.copy()
    k2[p + 1:] = rng.standard_normal(k2[p + 1:].shape)
    v2[p + 1:] = rng.standard_normal(v2[p + 1:].shape)
    b = run_sdpa(ctx, q, k2, v2, B, H, S, 0.125, True)
    assert (a[:p + 1].view(np.uint32) == b[:p + 1].view(np.uint32)).all()
    assert not (a[p + 1:] == b[p + 1:]).all()


def test_argument_checks(ctx):
    import mlfw_b200
    x = ctx.to_device(np.zeros((4, 4100), np.float32))
    g = ctx.to_device(np.zeros(4100, np.float32))
    with pytest.raises(mlfw_b200.B200QError):
        ctx.layernorm_quantize(x, None, g, g, 1e-5, 4, 4100)           # row too long
    with pytest.raises(mlfw_b200.B200QError):
        ctx.sdpa_f32(x, x, x, 128, 128, 128, 1, 2, 4, 32, 1.0, True, x, 128)   # head dimension


# ---------------------------------------------------------------------------------------------------------------
# The whole block, checked stage by stage: every stage of the oracle is fed what the device fed its own stage, so a
# code that flips on a tie inside one stage cannot masquerade as an error of the next.
# ---------------------------------------------------------------------------------------------------------------
def check_block_stages(ctx, orc, blk, params, h, B, S, rows=None):
    """rows: indices of the token rows to check (all when None)."""
    import mlfw_b200  # noqa: F401
    D, H, FF = blk.D, blk.H, blk.FF
    M = B * S
    dh = ctx.to_device(h)
    out = Guarded(ctx, (M, D), np.float32)
    t = blk.forward(dh, B, S, out.ptr)
    ctx.sync()
    ctx.check_status()
    got = {k: v.download() for k, v in t.items()}
    y = out.download()
    sel = np.arange(M) if rows is None else np.asarray(rows)

    def linear_ref(q, s, lin, act):
        w = lin.w.download()
        acc = orc.qdot_i32(q, w)
        return orc.epilogue(acc, s, lin.scales.download(), lin.bias.download(), act)

    # LayerNorm 1 + quantize
    n1 = orc.layer_norm(h[sel], params["ln1_gamma"], params["ln1_beta"], blk.eps)
    rq, _, rs = orc.quantize_per_token(n1)
    # the device quantizes ITS normalised values; they agree with the oracle's to tolerance, so compare dequantized rows
    deq_dev = got["n1_q"][sel].astype(np.float32) * got["n1_s"][sel][:, None]
    assert rel_err(deq_dev, n1) <= 1.0 / 127 + 1e-5
    # q/k/v projection from the device's own codes: bit-exact
    qkv_ref = linear_ref(got["n1_q"][sel], got["n1_s"][sel], blk.qkv, "none")
    assert (got["qkv"][sel].view(np.uint32) == qkv_ref.view(np.uint32)).all()
    # attention from the device's own projections
    qkv = got["qkv"]
    flat = [(b * H + hh) * S + i for m in sel[:64] for b, i in [divmod(int(m), S)] for hh in range(H)]
    a_ref = orc.sdpa(qkv[:, :D], qkv[:, D:2 * D], qkv[:, 2 * D:], B, H, S, 64, 1.0 / 8.0, True, rows=np.array(flat))
    a_dev = np.stack([got["attn"][(f // S // H) * S + f % S, ((f // S) % H) * 64:((f // S) % H + 1) * 64] for f in flat])
    assert rel_err(a_dev, a_ref) <= TOL
    # output projection: quantize the device's attention rows, then the linear
    aq, _, as_ = orc.quantize_per_token(got["attn"][sel])
    o_ref = linear_ref(aq, as_, blk.wo, "none")
    assert (got["o"][sel].view(np.uint32) == o_ref.view(np.uint32)).all()
    # residual + LayerNorm 2
    x_ref = h[sel] + got["o"][sel]
    assert (got["x"][sel].view(np.uint32) == x_ref.view(np.uint32)).all()
    n2 = orc.layer_norm(got["x"][sel], params["ln2_gamma"], params["ln2_beta"], blk.eps)
    deq2 = got["n2_q"][sel].astype(np.float32) * got["n2_s"][sel][:, None]
    assert rel_err(deq2, n2) <= 1.0 / 127 + 1e-5
    f1_ref = linear_ref(got["n2_q"][sel], got["n2_s"][sel], blk.fc1, blk.activation)
    assert (got["f1"][sel].view(np.uint32) == f1_ref.view(np.uint32)).all()
    fq, _, fs = orc.quantize_per_token(got["f1"][sel])
    f2_ref = linear_ref(fq, fs, blk.fc2, "none")
    assert (got["f2"][sel].view(np.uint32) == f2_ref.view(np.uint32)).all()
    assert (y[sel].view(np.uint32) == (got["x"][sel] + got["f2"][sel]).view(np.uint32)).all()
    return y


def test_block_small(ctx, orc):
    from mlfw_b200.block import GPTBlock, random_block_params
    D, H, FF, B, S = 128, 2, 512, 2, 96
    params = random_block_params(D, FF, seed=1, std=0.05)
    params["ln1_gamma"] = np.random.default_rng(2).uniform(0.5, 1.5, D).astype(np.float32)
    params["ln2_beta"] = np.random.default_rng(3).uniform(-0.2, 0.2, D).astype(np.float32)
    blk = GPTBlock(ctx, D, H, FF, params)
    h = np.random.default_rng(4).standard_normal((B * S, D)).astype(np.float32)
    y = check_block_stages(ctx, orc, blk, params, h, B, S)
    assert np.isfinite(y).all()


def test_block_config4_shape(ctx, orc):
    """d_model 768, 12 heads, ff 3072, 32 x 512 tokens: every stage checked on a sample of rows."""
    from mlfw_b200.block import GPTBlock, random_block_params
    D, H, FF, B, S = 768, 12, 3072, 32, 512
    params = random_block_params(D, FF, seed=7)
    blk = GPTBlock(ctx, D, H, FF, params)
    rng = np.random.default_rng(8)
    table = (rng.standard_normal((50257, D)) * 0.02).astype(np.float32)
    tokens = rng.integers(0, 50257, size=B * S).astype(np.int32)
    dh = ctx.empty((B * S, D), np.float32)
    ctx.embedding_f32(ctx.to_device(table), ctx.to_device(tokens), None, B * S, D, 50257, S, dh)
    ctx.sync()
    h = dh.download()
    assert (h.view(np.uint32) == table[tokens].view(np.uint32)).all()
    rows = np.unique(np.concatenate([[0, 1, 511, 512, 16383], rng.integers(0, B * S, size=27)]))
    check_block_stages(ctx, orc, blk, params, h, B, S, rows=rows)


def test_quantized_linear_survives_a_checkpoint(ctx):
    """int8 weights + scales + bias through the reference's checkpoint container and back: same device results."""
    from collections import OrderedDict
    from mlfw_b200.block import QuantLinear
    from mlfw_b200.checkpoint import deserialize_checkpoint, serialize_checkpoint
    rng = np.random.default_rng(21)
    N, K, M = 256, 512, 300
    lin = QuantLinear.from_float(ctx, (rng.standard_normal((N, K)) * 0.05).astype(np.float32), rng.standard_normal(N).astype(np.float32))
    blob = serialize_checkpoint({"epoch": 1, "modelState": OrderedDict([("fc", lin.state())])})
    lin2 = QuantLinear.from_state(ctx, deserialize_checkpoint(blob)["modelState"]["fc"])
    x = ctx.to_device(rng.standard_normal((M, K)).astype(np.float32))
    a, b = ctx.empty((M, N), np.float32), ctx.empty((M, N), np.float32)
    ctx.linear_f32(x, lin.w, lin.scales, lin.bias, "silu", M, N, K, a)
    ctx.linear_f32(x, lin2.w, lin2.scales, lin2.bias, "silu", M, N, K, b)
    ctx.sync()
    assert (a.download().view(np.uint32) == b.download().view(np.uint32)).all()

