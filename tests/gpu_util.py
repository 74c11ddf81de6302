"""Helpers of the GPU parity tests: guarded device buffers and seeded inputs."""
import numpy as np

MARGIN = 256  # bytes of canary on each side of a guarded buffer
PATTERN = 0xA5


class Guarded:
    """A device buffer with canary margins; ``check()`` fails if a kernel wrote outside its output."""

    def __init__(self, ctx, shape, dtype, fill=None):
        self.ctx = ctx
        self.shape = tuple(shape) if hasattr(shape, "__len__") else (shape,)
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        self.raw = ctx.empty(self.nbytes + 2 * MARGIN, np.uint8)
        self.raw.fill_bytes(PATTERN)
        self.ptr = self.raw.ptr + MARGIN
        if fill is not None:
            self.upload(fill)

    def upload(self, arr):
        a = np.ascontiguousarray(arr, self.dtype)
        assert a.nbytes == self.nbytes
        full = np.full(self.nbytes + 2 * MARGIN, PATTERN, np.uint8)
        full[MARGIN:MARGIN + self.nbytes] = a.view(np.uint8).reshape(-1)
        self.raw.upload(full)
        return self

    def download(self):
        full = self.raw.download()
        assert (full[:MARGIN] == PATTERN).all(), "kernel wrote before its output buffer"
        assert (full[MARGIN + self.nbytes:] == PATTERN).all(), "kernel wrote past its output buffer"
        return full[MARGIN:MARGIN + self.nbytes].view(self.dtype).reshape(self.shape).copy()


def activations(rng, M, K, outliers=True):
    x = rng.standard_normal((M, K)).astype(np.float32)
    if outliers and M * K > 16:
        mask = rng.random((M, K)) < 0.001
        x[mask] = (rng.standard_normal(int(mask.sum())) * 20).astype(np.float32)
    return x


def rel_err(a, b):
    """max |a-b| relative to the absmax of the expected tensor b (the tolerance the spec states)."""
    b = np.asarray(b, np.float64)
    a = np.asarray(a, np.float64)
    fin = np.isfinite(b)
    assert (np.isfinite(a) == fin).all()
    if not fin.any():
        return 0.0
    denom = np.abs(b[fin]).max()
    return float(np.abs(a[fin] - b[fin]).max() / (denom if denom > 0 else 1.0))
