"""Planner and host-side mirror of the multi-GPU forms of the quantized linear path.

The reference has no multi-device execution (its ``all_gather`` / ``all_reduce`` graph ops decompose to
single-device slices, src/compiler/passes/decompose/decomposition_pass.ts:105-143); this is new.  The execution
itself lives behind the C ABI (``b200q_group_*`` in ``include/b200q.h``, NCCL inside ``libb200q.so``); this module
holds what a host needs around it and what can be checked without a GPU:

* **Row (M) sharding** - every output row depends only on its own input row and the replicated weights, so the
  ranks take contiguous row blocks and nothing is exchanged on the data path (:func:`row_block`).
* **Column (N) sharding** - the weights are split by output channel, every rank holds the whole int8 activation.
  A layer is then: local GEMM + tail on the rank's columns; per-token requantization of the FULL row, which needs the
  row's range over all ranks (ONE max-reduction over order-preserving keys of the local minima and maxima,
  :func:`range_keys`) and then gives bit-identical codes on every rank; an all-gather of the int8 column blocks (int8
  on the wire, not f32).  :class:`ColumnShardedStack` states that protocol against a small compute interface, so
  that it runs on CPU ranks (gloo) in the tests with a CPU stand-in for the kernels.
* The layout ``b200q_group_linear_nshard`` leaves its gathered codes in (:func:`chunk_rows`,
  :func:`from_gathered_layout`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np


def row_block(M: int, world: int, rank: int) -> Tuple[int, int]:
    """(first row, row count) of ``rank``: contiguous blocks, the first ``M % world`` ranks take one row more."""
    base, extra = divmod(M, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def column_block(N: int, world: int, rank: int, align: int = 256) -> Tuple[int, int]:
    """(first column, column count) of ``rank``: whole ``align``-wide tiles are dealt out as evenly as possible, the
    ragged remainder of N goes to the last rank that has any columns."""
    tiles = (N + align - 1) // align
    base, extra = divmod(tiles, world)
    t0 = rank * base + min(rank, extra)
    t1 = t0 + base + (1 if rank < extra else 0)
    start, stop = min(t0 * align, N), min(t1 * align, N)
    return start, stop - start


@dataclass
class ShardedLayer:
    """One int8 linear of a column-sharded stack, as held by one rank."""
    K: int
    N: int                      # full output width
    col0: int                   # this rank's first output channel
    cols: int                   # and how many it owns
    w: object                   # int8 [cols, K] (K-major rows of the rank's channels)
    w_scales: object            # f32 [cols]
    bias: Optional[object]      # f32 [cols] or None
    act: str


class ColumnShardedStack:
    """Runs consecutive int8 linears with per-token requantization between them, weights split by output channel.

    ``ops`` supplies the computation on one rank (the tests pass a CPU stand-in); ``dist`` is ``torch.distributed`` (or
    None for a single rank).  Activations travel between layers as int8 codes [M, N] plus f32 scales [M], identical
    on every rank."""

    def __init__(self, ops, dist, rank: int, world: int, layers: Sequence[ShardedLayer]):
        self.ops, self.dist, self.rank, self.world, self.layers = ops, dist, rank, world, list(layers)

    def forward(self, q, scales, M: int, last_f32: bool = True):
        """q int8 [M, K0], scales f32 [M] (replicated).  Returns (codes, scales) of the last layer, or its f32 output
        gathered over the ranks when ``last_f32``."""
        ops = self.ops
        for li, layer in enumerate(self.layers):
            y = ops.linear(q, scales, layer, M)                       # f32 [M, cols] on this rank
            final = li == len(self.layers) - 1
            if final and last_f32:
                return ops.all_gather_columns(y, M, layer, self.dist, self.world, np.float32), None
            mn, mx = ops.row_range(y, M, layer.cols)
            keys = ops.to_keys(mn, mx)                                # [2*M] order-preserving keys, 0 = nothing seen
            if self.dist is not None and self.world > 1:              # the exchange step: ONE max-reduction over all ranks
                ops.all_reduce_max(keys, self.dist)
            mn, mx = ops.from_keys(keys)
            q_local, scales = ops.quantize_with_range(y, M, layer.cols, mn, mx)
            q = ops.all_gather_columns(q_local, M, layer, self.dist, self.world, np.int8)   # int8 on the wire
        return q, scales


def gather_layout(N: int, world: int, align: int = 256) -> List[Tuple[int, int]]:
    """Column blocks of all ranks, in rank order (what the gathered pieces have to be laid out as)."""
    return [column_block(N, world, r, align) for r in range(world)]


def range_keys(mn: np.ndarray, mx: np.ndarray) -> np.ndarray:
    """Order-preserving uint32 keys of per-row minima and maxima, as the GEMM epilogue publishes them: ``[0, M)`` the
    maxima (a key grows with the value), ``[M, 2M)`` the minima (a key grows as the value falls), 0 where nothing was
    seen (``mx = -inf`` / ``mn = +inf``, or NaN).  The maximum of two ranks' keys is the key of their joint range."""
    def key_max(v):
        u = np.ascontiguousarray(v, np.float32).view(np.uint32)
        k = np.where(u & np.uint32(0x80000000), ~u, u | np.uint32(0x80000000)).astype(np.uint32)
        return k
    mn, mx = np.asarray(mn, np.float32), np.asarray(mx, np.float32)
    kmax = np.where(np.isnan(mx) | (mx == -np.inf), np.uint32(0), key_max(mx))
    kmin = np.where(np.isnan(mn) | (mn == np.inf), np.uint32(0), ~key_max(mn))
    return np.concatenate([kmax, kmin]).astype(np.uint32)


def range_from_keys(keys: np.ndarray):
    """(minima, maxima) f32 from :func:`range_keys` output; 0 decodes to +inf / -inf."""
    keys = np.asarray(keys, np.uint32)
    M = keys.size // 2

    def val_max(k):
        u = np.where(k & np.uint32(0x80000000), k & np.uint32(0x7FFFFFFF), ~k).astype(np.uint32)
        return u.view(np.float32)
    kmax, kmin = keys[:M], keys[M:]
    mx = np.where(kmax == 0, np.float32(-np.inf), val_max(kmax)).astype(np.float32)
    mn = np.where(kmin == 0, np.float32(np.inf), val_max(~kmin)).astype(np.float32)
    return mn, mx


def chunk_rows(M: int, chunks: int, c: int) -> Tuple[int, int]:
    """(first row, rows) of row chunk ``c`` of the column-sharded call: whole 256-row tiles, the last takes the rest."""
    per = ((M + chunks - 1) // chunks + 255) // 256 * 256
    a, b = min(per * c, M), min(per * (c + 1), M)
    return a, b - a


def from_gathered_layout(buf: np.ndarray, M: int, N: int, world: int, chunks: int = 1) -> np.ndarray:
    """Row-major ``[M, N]`` from the layout ``b200q_group_linear_nshard`` leaves its gathered codes in: per row chunk
    (starting at element ``N * first_row``) the ranks' column blocks one after the other, block ``r`` a row-major
    ``[rows of the chunk, N / world]`` matrix."""
    cols = N // world
    flat = np.asarray(buf).reshape(-1)
    out = np.empty((M, N), flat.dtype)
    for c in range(chunks):
        r0, rows = chunk_rows(M, chunks, c)
        if rows == 0:
            continue
        blk = flat[r0 * N:(r0 + rows) * N].reshape(world, rows, cols)
        for r in range(world):
            out[r0:r0 + rows, r * cols:(r + 1) * cols] = blk[r]
    return out


def to_gathered_layout(a: np.ndarray, world: int, chunks: int = 1) -> np.ndarray:
    """Inverse of :func:`from_gathered_layout` (flat array of ``M * N`` elements)."""
    M, N = a.shape
    cols = N // world
    out = np.empty(M * N, a.dtype)
    for c in range(chunks):
        r0, rows = chunk_rows(M, chunks, c)
        if rows == 0:
            continue
        out[r0 * N:(r0 + rows) * N] = np.stack([a[r0:r0 + rows, r * cols:(r + 1) * cols] for r in range(world)]).reshape(-1)
    return out


def gather_columns(torch, dist, local, M: int, N: int, world: int):
    """All-gather of column blocks [M, cols_r] into [M, N].  Blocks may differ in width: every rank sends a piece
    padded to the widest block (one collective, equal sizes), the padding is dropped when the row-major result is
    assembled."""
    blocks = gather_layout(N, world)
    widest = max(c for _, c in blocks)
    piece = local
    if local.shape[1] != widest:
        piece = torch.zeros((M, widest), dtype=local.dtype, device=local.device)
        piece[:, : local.shape[1]] = local
    flat = torch.empty((world * M, widest), dtype=local.dtype, device=local.device)   # rank r's piece lands in rows [r*M, (r+1)*M)
    dist.all_gather_into_tensor(flat, piece.contiguous())
    gathered = flat.view(world, M, widest)
    return torch.cat([gathered[r, :, :c] for r, (_, c) in enumerate(blocks) if c > 0], dim=1).contiguous()
