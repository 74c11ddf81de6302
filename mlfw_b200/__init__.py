"""mlfw_b200 — B200 backend for mlfw's int8 quantized-inference path.

``libb200q.so`` (hand-written CUDA for sm_100a behind a C ABI, ``include/b200q.h``)
is the product; this package is its Python host side: the ctypes binding, a thin
object layer, and the mirror of the reference's backend interface
(:mod:`mlfw_b200.backend`).  There is no CPU fallback.
"""
from ._lib import B200QError, LIB_PATH
from .device import ACT, Context, DeviceBuffer, Group, PinnedArray, W_KN, W_NK

__all__ = ["B200QError", "LIB_PATH", "ACT", "Context", "DeviceBuffer", "Group", "PinnedArray", "W_KN", "W_NK"]
