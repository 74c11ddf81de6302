"""GPU parity of the quantize / dequantize kernels against the CPU oracle (through the C ABI).

int8 codes and scales must be bit-exact; f32 results are bit-exact against the oracle
evaluated with the same binary32 scales and within 1e-5 of the output absmax against
the reference's binary64-scale arithmetic.
"""
import numpy as np
import pytest

from gpu_util import Guarded, activations, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5  # max-abs relative to output absmax


@pytest.fixture(scope="module")
def ctx():
    import mlfw_b200
    c = mlfw_b200.Context(0)
    yield c
    c.check_status()
    c.close()


def run_quantize_per_token(ctx, x, qmin=-127, qmax=127):
    M, K = x.shape
    dx = Guarded(ctx, (M, K), np.float32, x)
    dq = Guarded(ctx, (M, K), np.int8)
    ds = Guarded(ctx, (M,), np.float32)
    ctx.quantize_per_token(dx.ptr, M, K, dq.ptr, ds.ptr, qmin, qmax)
    ctx.sync()
    return dq.download(), ds.download()


SHAPES = [(1, 1), (3, 5), (2, 6), (7, 64), (33, 128), (256, 512), (5, 768), (9, 3072), (4, 4096), (17, 4100),
          (3, 8192), (2, 28672), (2, 32772), (1, 40000), (300, 4),
          # 64 rows or more: the shared-memory staged kernel (variant 0) unless a row exceeds 32 KB
          (100, 768), (65, 3072), (64, 8192), (70, 4096), (333, 512), (64, 4100), (1000, 16), (129, 2052), (200, 2048),
          # many chunks per block: every ring of slots wraps several times
          (6000, 4096), (40000, 512), (20011, 768)]


# variant 0: rows staged in shared memory when they fit (rows of 8, 12 and 16 KB are then moved into registers and their
# slot handed back early); 1: unstaged kernel only; 2: staged, both passes from shared memory for every row length
@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("M,K", SHAPES)
def test_quantize_per_token_bit_exact(ctx, orc, M, K, variant):
    rng = np.random.default_rng(M * 100003 + K)
    x = activations(rng, M, K)
    ctx.set_quant_variant(variant)
    try:
        q, s = run_quantize_per_token(ctx, x)
    finally:
        ctx.set_quant_variant(0)
    rq, _, rs32 = orc.quantize_per_token(x)
    assert (s.view(np.uint32) == rs32.view(np.uint32)).all()
    assert (q == rq).all(), f"{int((q != rq).sum())} codes differ"


def test_quantize_per_token_special_rows(ctx, orc):
    K = 64
    rows = []
    rows.append(np.zeros(K, np.float32))                                   # all zero: range widened to +-0.5
    rows.append(np.full(K, 3.0, np.float32))                               # all equal
    r = np.linspace(-2, 2, K).astype(np.float32); r[5] = np.nan; rows.append(r)      # NaN ignored, code 0
    r = np.linspace(-4, 1, K).astype(np.float32); r[7] = np.inf; rows.append(r)      # +Inf: max -> 1
    r = np.linspace(-1, 3, K).astype(np.float32); r[9] = -np.inf; rows.append(r)     # -Inf: min -> -1
    rows.append(np.full(K, np.nan, np.float32))                            # nothing finite
    rows.append((np.linspace(-1, 1, K) * 1e-41).astype(np.float32))        # denormals: reciprocal overflows binary32
    rows.append((np.linspace(-1, 1, K) * 3e38).astype(np.float32))         # huge
    r = np.zeros(K, np.float32); r[3] = -0.0; r[4] = 1e-45; rows.append(r)
    r = np.full(K, -7.25, np.float32); rows.append(r)                      # all equal, negative
    x = np.stack(rows)
    x = np.concatenate([x] * 7)          # 70 rows: the staged kernel takes them too
    for qmin, qmax in [(-127, 127), (-128, 127), (-100, 100)]:
        q, s = run_quantize_per_token(ctx, x, qmin, qmax)
        rq, _, rs32 = orc.quantize_per_token(x, qmin, qmax)
        assert (s.view(np.uint32) == rs32.view(np.uint32)).all()
        assert (q == rq).all()


def test_quantize_per_token_constructed_ties(ctx, orc):
    """Inputs built by inverting the map: x = (k + 0.5) * scale, one ulp either side included."""
    rng = np.random.default_rng(7)
    rows = []
    for absmax in [1.0, 3.0, 127.0, 6.0, 0.37, 1e-3, 254.0, 5.5, float(np.float32(2.0 / 3.0)), 1e20]:
        s = np.float64(np.float32(absmax)) / 127.0
        ks = rng.integers(-127, 127, size=253).astype(np.float64)
        base = ((ks + 0.5) * s).astype(np.float32)
        up = np.nextafter(base, np.float32(np.inf))
        dn = np.nextafter(base, np.float32(-np.inf))
        row = np.concatenate([[np.float32(absmax)], base, up, dn]).astype(np.float32)
        rows.append(row)
    x = np.stack(rows)
    x = np.concatenate([x] * 7)          # 70 rows: the staged kernel
    x = np.clip(x, -np.abs(x[:, :1]), np.abs(x[:, :1]))  # keep the first entry the absmax
    q, s = run_quantize_per_token(ctx, x)
    rq, _, rs32 = orc.quantize_per_token(x)
    assert (s.view(np.uint32) == rs32.view(np.uint32)).all()
    assert (q == rq).all(), f"{int((q != rq).sum())} tie codes differ"


@pytest.mark.parametrize("variant", [0, 2])
@pytest.mark.parametrize("K", [2048, 3072, 4096])
def test_quantize_per_token_long_rows_special_and_ties(ctx, orc, K, variant):
    """Row lengths that take the register-resident form of the staged kernel: odd rows (NaN, infinities, constant,
    denormal, huge), constructed ties with their neighbours, and ordinary rows in between, many rows per block."""
    rng = np.random.default_rng(K)
    rows = []
    for rep in range(40):
        rows.append(rng.standard_normal(K).astype(np.float32) * np.float32(10.0 ** rng.integers(-3, 4)))
        r = rng.standard_normal(K).astype(np.float32); r[rng.integers(0, K, 5)] = np.nan; rows.append(r)
        r = rng.standard_normal(K).astype(np.float32); r[rng.integers(0, K)] = np.inf; rows.append(r)
        r = rng.standard_normal(K).astype(np.float32); r[rng.integers(0, K)] = -np.inf; rows.append(r)
        rows.append(np.full(K, np.float32(rng.standard_normal()), np.float32))
        rows.append((rng.uniform(-1, 1, K) * 1e-41).astype(np.float32))
        rows.append((rng.uniform(-1, 1, K) * 3e38).astype(np.float32))
        absmax = np.float32([1.0, 3.0, 127.0, 6.0, 0.37, 1e-3, 254.0, 5.5, 2.0 / 3.0, 1e20][rep % 10])
        sc = np.float64(absmax) / 127.0
        ks = rng.integers(-127, 127, size=(K - 1) // 3).astype(np.float64)
        base = ((ks + 0.5) * sc).astype(np.float32)
        row = np.concatenate([[absmax], base, np.nextafter(base, np.float32(np.inf)), np.nextafter(base, np.float32(-np.inf))])
        row = np.concatenate([row, np.zeros(K - row.size)]).astype(np.float32)
        rows.append(np.clip(row, -absmax, absmax))
    rows.append(np.full(K, np.nan, np.float32))
    rows.append(np.zeros(K, np.float32))
    x = np.stack(rows)
    ctx.set_quant_variant(variant)
    try:
        for qmin, qmax in [(-127, 127), (-128, 127), (-100, 100)]:
            q, s = run_quantize_per_token(ctx, x, qmin, qmax)
            rq, _, rs32 = orc.quantize_per_token(x, qmin, qmax)
            assert (s.view(np.uint32) == rs32.view(np.uint32)).all()
            assert (q == rq).all(), f"{int((q != rq).sum())} codes differ"
    finally:
        ctx.set_quant_variant(0)
    ctx.check_status()


@pytest.mark.parametrize("M,K", [(1, 1), (3, 5), (33, 128), (5, 768), (4, 4096), (17, 4100), (2, 28672), (300, 4)])
def test_dequantize_per_token(ctx, orc, M, K):
    rng = np.random.default_rng(M * 7 + K)
    x = activations(rng, M, K)
    rq, s64, rs32 = orc.quantize_per_token(x)
    dq = Guarded(ctx, (M, K), np.int8, rq)
    ds = Guarded(ctx, (M,), np.float32, rs32)
    dy = Guarded(ctx, (M, K), np.float32)
    ctx.dequantize_per_token(dq.ptr, ds.ptr, M, K, dy.ptr)
    ctx.sync()
    y = dy.download()
    ref32 = orc.dequantize_per_token_f32(rq, rs32)
    assert (y.view(np.uint32) == ref32.view(np.uint32)).all()
    ref64 = orc.dequantize_per_channel(rq, (M, K), 0, s64)   # the reference's binary64 arithmetic
    assert rel_err(y, ref64) <= TOL


def test_roundtrip_error_bound(ctx, orc):
    """quantize -> dequantize stays within half a step per element (params.test.js:166-176 applied per token)."""
    rng = np.random.default_rng(11)
    M, K = 64, 1024
    x = activations(rng, M, K)
    q, s = run_quantize_per_token(ctx, x)
    dq = Guarded(ctx, (M, K), np.int8, q)
    ds = Guarded(ctx, (M,), np.float32, s)
    dy = Guarded(ctx, (M, K), np.float32)
    ctx.dequantize_per_token(dq.ptr, ds.ptr, M, K, dy.ptr)
    ctx.sync()
    y = dy.download()
    assert (np.abs(y.astype(np.float64) - x) <= s[:, None].astype(np.float64) / 2 * (1 + 1e-6) + 1e-9).all()


STATIC_SCALES = [6 / 127, 0.02, 0.05, 0.5, 1.0, 3 / 127, 1e-3, 7.0]


@pytest.mark.parametrize("n", [1, 3, 4, 17, 1024, 4099, 1 << 16])
def test_quantize_static(ctx, orc, n):
    rng = np.random.default_rng(n)
    for scale in STATIC_SCALES:
        x = (rng.standard_normal(n) * 60 * scale).astype(np.float32)
        # every fourth element sits on (or one ulp around) a rounding tie of fround(x/scale)
        k = rng.integers(-130, 130, size=n).astype(np.float64)
        tie = ((k + 0.5) * scale).astype(np.float32)
        tie = np.where(np.arange(n) % 3 == 0, np.nextafter(tie, np.float32(np.inf)), tie)
        tie = np.where(np.arange(n) % 3 == 1, np.nextafter(tie, np.float32(-np.inf)), tie)
        x = np.where(np.arange(n) % 4 == 0, tie, x).astype(np.float32)
        for zp, kind in [(0, 0), (0, 1), (5, 0), (128, 1), (-3, 0)]:
            dx = Guarded(ctx, (n,), np.float32, x)
            dq = Guarded(ctx, (n,), np.int8)
            ctx.quantize_static(dx.ptr, n, scale, zp, kind, dq.ptr)
            ctx.sync()
            q = dq.download()
            ref = orc.quantize_static(x, scale, zp, kind).view(np.int8)
            assert (q == ref).all(), f"scale={scale} zp={zp} kind={kind}: {int((q != ref).sum())} differ"


def test_quantize_static_special_values(ctx, orc):
    x = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1e30, -1e30, 3e38, 1e-45, -1e-45, 2.5 * 6 / 127], np.float32)
    for scale in [6 / 127, 1e-30, 1e30, 1e-42, -0.05]:
        dx = Guarded(ctx, x.shape, np.float32, x)
        dq = Guarded(ctx, x.shape, np.int8)
        ctx.quantize_static(dx.ptr, x.size, scale, 0, 0, dq.ptr)
        ctx.sync()
        assert (dq.download() == orc.quantize_static(x, scale, 0, 0)).all(), f"scale {scale}"


@pytest.mark.parametrize("n", [1, 5, 64, 4099, 1 << 16])
def test_dequantize_static(ctx, orc, n):
    rng = np.random.default_rng(n + 1)
    for scale in STATIC_SCALES:
        for zp in [0, 3, -7]:
            q8 = rng.integers(-128, 128, size=n).astype(np.int8)
            u8 = rng.integers(0, 256, size=n).astype(np.uint8)
            i32 = rng.integers(-2 ** 31, 2 ** 31 - 1, size=n).astype(np.int32)
            i32[: min(n, 8)] = [0, 1, -1, 2 ** 24, 2 ** 24 + 1, -(2 ** 31), 2 ** 31 - 1, 12345][: min(n, 8)]
            for arr, kind in [(q8, 0), (u8, 1), (i32, 2)]:
                dq = Guarded(ctx, (n,), arr.dtype, arr)
                dy = Guarded(ctx, (n,), np.float32)
                ctx.dequantize_static(dq.ptr, kind, n, scale, zp, dy.ptr)
                ctx.sync()
                y = dy.download()
                ref = orc.dequantize_static(arr, scale, zp)
                assert (y.view(np.uint32) == ref.view(np.uint32)).all(), f"kind={kind} scale={scale} zp={zp}"


@pytest.mark.parametrize("N,K,layout", [(6, 8, 1), (3, 4, 1), (64, 128, 0), (33, 70, 0), (33, 70, 1), (1024, 512, 1), (256, 1024, 0)])
def test_quantize_weights_per_channel(ctx, orc, N, K, layout):
    """quantization_pass.ts:390-400: per-output-channel scales and codes, emitted K-major."""
    rng = np.random.default_rng(N * 31 + K)
    w_nk = (rng.standard_normal((N, K)) * 0.02 * (1 + np.arange(N))[:, None]).astype(np.float32)
    if N > 4:
        w_nk[2] = 0.0          # constant channel
        w_nk[3] = 0.125
    src = w_nk if layout == 0 else np.ascontiguousarray(w_nk.T)   # [N,K] or [K,N]
    dw = Guarded(ctx, src.shape, np.float32, src)
    dq = Guarded(ctx, (N, K), np.int8)
    ds32 = Guarded(ctx, (N,), np.float32)
    ds64 = Guarded(ctx, (N,), np.float64)
    ctx.quantize_weights_per_channel(dw.ptr, N, K, layout, dq.ptr, ds32.ptr, ds64.ptr)
    ctx.sync()
    axis = 0 if layout == 0 else 1
    rs = orc.per_channel_scales(src, src.shape, axis)
    rq = orc.quantize_per_channel(src, src.shape, axis, rs, -128, 127)
    rq_nk = rq if layout == 0 else np.ascontiguousarray(rq.T)
    assert (ds64.download() == rs).all()
    assert (ds32.download() == rs.astype(np.float32)).all()
    assert (dq.download() == rq_nk).all()


def test_transpose_i8(ctx):
    rng = np.random.default_rng(5)
    for K, N in [(1, 1), (5, 3), (64, 33), (100, 257)]:
        w = rng.integers(-128, 128, size=(K, N)).astype(np.int8)
        d_in = Guarded(ctx, (K, N), np.int8, w)
        d_out = Guarded(ctx, (N, K), np.int8)
        ctx.transpose_i8(d_in.ptr, K, N, d_out.ptr)
        ctx.sync()
        assert (d_out.download() == w.T).all()


def test_empty_inputs_are_noops(ctx):
    ctx.quantize_per_token(None, 0, 128, None, None)
    ctx.dequantize_per_token(None, None, 0, 128, None)
    ctx.quantize_static(None, 0, 0.05, 0, 0, None)
    ctx.dequantize_static(None, 0, 0, 0.05, 0, None)
    ctx.sync()


def test_argument_errors(ctx):
    import mlfw_b200
    d = ctx.empty((4, 4), np.float32)
    with pytest.raises(mlfw_b200.B200QError):
        ctx.quantize_per_token(d.ptr, 4, 4, None, None)           # null outputs
    with pytest.raises(mlfw_b200.B200QError):
        ctx.quantize_per_token(d.ptr, -1, 4, d.ptr, d.ptr)        # negative dimension
    with pytest.raises(mlfw_b200.B200QError):
        ctx.quantize_static(d.ptr, 16, 0.0, 0, 0, d.ptr)          # zero scale
    with pytest.raises(mlfw_b200.B200QError):
        ctx.quantize_static(d.ptr, 16, 0.1, 0, 2, d.ptr)          # int32 is not a quantize target
    with pytest.raises(mlfw_b200.B200QError):
        ctx.quantize_per_token(d.ptr, 4, 4, d.ptr, d.ptr, -200, 127)
