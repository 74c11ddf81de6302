"""Multi-GPU host logic of the quantized linear path (one process per GPU, ``torch.distributed`` for the plumbing).

The reference has no multi-device execution (its ``all_gather`` / ``all_reduce`` graph ops decompose to
single-device slices, src/compiler/passes/decompose/decomposition_pass.ts:105-143); this is new.

* **Row (M) sharding** — every output row depends only on its own input row and the replicated weights, so the
  ranks take contiguous row blocks and nothing is exchanged on the data path (:func:`row_block`).
* **Column (N) sharding** — the weights are split by output channel, every rank holds the whole int8 activation.
  A layer is then: local GEMM + tail on the rank's columns; per-token requantization of the FULL row, which needs the
  row's range over all ranks (two tiny all-reduces, min and max) and then gives bit-identical codes on every
  rank; an all-gather of the int8 column blocks (int8 on the wire, not f32).  :class:`ColumnShardedStack` runs a
  stack of such layers.  It is written against a small compute interface so that the collective logic runs on CPU
  ranks (gloo) in the tests with a CPU stand-in, and on GPUs with :class:`DeviceOps`.
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

    ``ops`` supplies the computation on one rank (see :class:`DeviceOps`); ``dist`` is ``torch.distributed`` (or
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
            if self.dist is not None and self.world > 1:              # the exchange step: row ranges over all ranks
                ops.all_reduce(mn, "min", self.dist)
                ops.all_reduce(mx, "max", self.dist)
            q_local, scales = ops.quantize_with_range(y, M, layer.cols, mn, mx)
            q = ops.all_gather_columns(q_local, M, layer, self.dist, self.world, np.int8)   # int8 on the wire
        return q, scales


def gather_layout(N: int, world: int, align: int = 256) -> List[Tuple[int, int]]:
    """Column blocks of all ranks, in rank order (what the gathered pieces have to be laid out as)."""
    return [column_block(N, world, r, align) for r in range(world)]


class DeviceOps:
    """The compute interface of :class:`ColumnShardedStack` on one GPU: torch CUDA tensors hold the buffers (so NCCL can
    move them), every computation is a call into libb200q.so on the context's stream."""

    def __init__(self, ctx, torch):
        self.ctx, self.torch = ctx, torch
        self.dev = torch.device("cuda", ctx.device)

    def _sync_in(self):                 # torch work (collectives, copies) before library kernels
        self.torch.cuda.current_stream(self.dev).synchronize()

    def _sync_out(self):                # library kernels before torch work
        self.ctx.sync()

    def linear(self, q, scales, layer: ShardedLayer, M: int):
        t = self.torch
        y = t.empty((M, layer.cols), dtype=t.float32, device=self.dev)
        self._sync_in()
        self.ctx.int8_linear(q.data_ptr(), scales.data_ptr(), layer.w.data_ptr(), layer.w_scales.data_ptr(),
                             layer.bias.data_ptr() if layer.bias is not None else None, layer.act, M, layer.cols, layer.K, y.data_ptr())
        self._sync_out()
        return y

    def row_range(self, y, M: int, cols: int):
        t = self.torch
        mn = t.empty((M,), dtype=t.float32, device=self.dev)
        mx = t.empty((M,), dtype=t.float32, device=self.dev)
        self._sync_in()
        self.ctx.row_range(y.data_ptr(), M, cols, cols, mn.data_ptr(), mx.data_ptr())
        self._sync_out()
        return mn, mx

    def all_reduce(self, v, op: str, dist):
        dist.all_reduce(v, op=dist.ReduceOp.MIN if op == "min" else dist.ReduceOp.MAX)

    def quantize_with_range(self, y, M: int, cols: int, mn, mx):
        t = self.torch
        q = t.empty((M, cols), dtype=t.int8, device=self.dev)
        s = t.empty((M,), dtype=t.float32, device=self.dev)
        self._sync_in()
        self.ctx.quantize_rows_with_range(y.data_ptr(), M, cols, cols, mn.data_ptr(), mx.data_ptr(), q.data_ptr(), cols, s.data_ptr())
        self._sync_out()
        return q, s

    def all_gather_columns(self, local, M: int, layer: ShardedLayer, dist, world: int, dtype):
        if dist is None or world == 1:
            return local
        return gather_columns(self.torch, dist, local, M, layer.N, world)


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
