"""Thin object layer over the C ABI: a context per GPU, device buffers, the ops.

numpy arrays are the host side (the reference hands its backends typed arrays,
src/runtime/runtime.ts:239-259); device memory belongs to the library.  Nothing
here computes: every method is one call into ``libb200q.so``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import B200QError, check

ACT = {"none": 0, "relu": 1, "gelu_sigmoid": 2, "gelu_tanh": 3, "silu": 4}
W_NK, W_KN = 0, 1
KIND = {np.dtype(np.int8): 0, np.dtype(np.uint8): 1, np.dtype(np.int32): 2}

STATUS_BITS = {1: "TMA producer wait ran out", 2: "MMA issuer wait ran out", 4: "epilogue wait ran out",
               8: "unexpected tensor-memory allocation", 16: "staged quantize wait ran out"}


class DeviceBuffer:
    """Device memory with a dtype and shape attached for convenience."""

    def __init__(self, ctx: "Context", shape, dtype):
        self.ctx = ctx
        self.shape = tuple(int(s) for s in (shape if hasattr(shape, "__len__") else (shape,)))
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        p = C.c_void_p()
        check(ctx.lib.b200q_alloc(ctx.handle, self.nbytes, C.byref(p)), "b200q_alloc")
        self.ptr = p.value
        self._free = True

    def upload(self, arr) -> "DeviceBuffer":
        a = np.ascontiguousarray(arr, dtype=self.dtype)
        if a.nbytes != self.nbytes:
            raise ValueError(f"upload of {a.nbytes} bytes into a buffer of {self.nbytes}")
        check(self.ctx.lib.b200q_upload(self.ctx.handle, self.ptr, a.ctypes.data, a.nbytes), "b200q_upload")
        return self

    def download(self) -> np.ndarray:
        out = np.empty(self.shape, self.dtype)
        check(self.ctx.lib.b200q_download(self.ctx.handle, out.ctypes.data, self.ptr, self.nbytes), "b200q_download")
        return out

    def fill_bytes(self, value: int) -> "DeviceBuffer":
        check(self.ctx.lib.b200q_memset(self.ctx.handle, self.ptr, value, self.nbytes), "b200q_memset")
        return self

    def free(self) -> None:
        if self._free and self.ptr is not None and self.ctx.handle:
            self.ctx.lib.b200q_free(self.ctx.handle, self.ptr)
        self._free = False
        self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class PinnedArray:
    """Page-locked host memory viewed as a numpy array (for the host-buffer entry points)."""

    def __init__(self, ctx: "Context", shape, dtype):
        self.ctx = ctx
        self.dtype = np.dtype(dtype)
        self.shape = tuple(int(s) for s in (shape if hasattr(shape, "__len__") else (shape,)))
        n = int(np.prod(self.shape, dtype=np.int64))
        p = C.c_void_p()
        check(ctx.lib.b200q_host_alloc(ctx.handle, n * self.dtype.itemsize, C.byref(p)), "b200q_host_alloc")
        self.ptr = p.value
        buf = (C.c_char * (n * self.dtype.itemsize)).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=self.dtype, count=n).reshape(self.shape)

    def free(self):
        if self.ptr is not None and self.ctx.handle:
            self.array = None
            self.ctx.lib.b200q_host_free(self.ctx.handle, self.ptr)
        self.ptr = None


def _ptr(b):
    if b is None:
        return None
    if isinstance(b, (DeviceBuffer, PinnedArray)):
        return b.ptr
    if isinstance(b, np.ndarray):
        return b.ctypes.data
    return int(b)  # raw address (e.g. torch.Tensor.data_ptr())


class Context:
    """One GPU.  Raises if no CUDA device (or the library) is available."""

    def __init__(self, device: int = 0):
        self.lib = _lib.lib()
        h = C.c_void_p()
        check(self.lib.b200q_create(device, C.byref(h)), "b200q_create")
        self.handle = h.value
        self.device = device

    def close(self):
        if self.handle:
            self.lib.b200q_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # ---- plumbing
    def empty(self, shape, dtype) -> DeviceBuffer:
        return DeviceBuffer(self, shape, dtype)

    def to_device(self, arr) -> DeviceBuffer:
        a = np.ascontiguousarray(arr)
        return DeviceBuffer(self, a.shape, a.dtype).upload(a)

    def pinned(self, shape, dtype) -> PinnedArray:
        return PinnedArray(self, shape, dtype)

    def sync(self):
        check(self.lib.b200q_sync(self.handle), "b200q_sync")

    def status_word(self) -> int:
        v = C.c_uint32()
        check(self.lib.b200q_status_word(self.handle, C.byref(v)), "b200q_status_word")
        return v.value

    def check_status(self):
        s = self.status_word()
        if s:
            names = [n for b, n in STATUS_BITS.items() if s & b]
            raise B200QError(f"device status word is {s:#x}: {', '.join(names)}")

    def clear_status(self):
        check(self.lib.b200q_clear_status(self.handle), "b200q_clear_status")

    def set_wait_limit(self, seconds: float):
        check(self.lib.b200q_set_wait_limit(self.handle, seconds), "b200q_set_wait_limit")

    def set_gemm_variant(self, variant: int):
        check(self.lib.b200q_set_gemm_variant(self.handle, variant), "b200q_set_gemm_variant")

    def set_tail_mode(self, mode: int):
        """0: exact sigmoid tails (default); 1: hardware exp / reciprocal for f32 outputs (within the 1e-5 bar, faster)."""
        check(self.lib.b200q_set_tail_mode(self.handle, mode), "b200q_set_tail_mode")

    def set_quant_variant(self, variant: int):
        check(self.lib.b200q_set_quant_variant(self.handle, variant), "b200q_set_quant_variant")

    def launch_count(self) -> int:
        return int(self.lib.b200q_launch_count(self.handle))

    def sm_count(self) -> int:
        return int(self.lib.b200q_sm_count(self.handle))

    def timer_start(self):
        check(self.lib.b200q_timer_start(self.handle), "b200q_timer_start")

    def timer_stop(self) -> float:
        ms = C.c_float()
        check(self.lib.b200q_timer_stop(self.handle, C.byref(ms)), "b200q_timer_stop")
        return ms.value

    KERNEL_KINDS = ("quantize_per_token", "dequantize_per_token", "quantize_static", "dequantize_static", "weights",
                    "gemm_tensor_core", "gemm_cuda_core", "tail", "embedding", "layernorm_quantize", "sdpa", "add")

    def profile_enable(self, on: bool = True):
        check(self.lib.b200q_profile_enable(self.handle, int(on)), "b200q_profile_enable")

    def profile_reset(self):
        check(self.lib.b200q_profile_reset(self.handle), "b200q_profile_reset")

    def profile_read(self) -> dict:
        """{kernel family: (total ms, launches)} since the last reset (synchronises)."""
        out = {}
        for k, name in enumerate(self.KERNEL_KINDS):
            ms, n = C.c_double(), C.c_uint64()
            check(self.lib.b200q_profile_read(self.handle, k, C.byref(ms), C.byref(n)), "b200q_profile_read")
            if n.value:
                out[name] = (ms.value, int(n.value))
        return out

    # ---- ops (device pointers)
    def quantize_per_token(self, x, M, K, q, scales, qmin=-127, qmax=127):
        check(self.lib.b200q_quantize_per_token(self.handle, _ptr(x), M, K, _ptr(q), _ptr(scales), qmin, qmax),
              "b200q_quantize_per_token")

    def dequantize_per_token(self, q, scales, M, K, y):
        check(self.lib.b200q_dequantize_per_token(self.handle, _ptr(q), _ptr(scales), M, K, _ptr(y)),
              "b200q_dequantize_per_token")

    def row_range(self, y, M, N, ld, row_min, row_max):
        check(self.lib.b200q_row_range(self.handle, _ptr(y), M, N, ld, _ptr(row_min), _ptr(row_max)), "b200q_row_range")

    def quantize_rows_with_range(self, y, M, N, ld_in, row_min, row_max, q, ld_out, scales, qmin=-127, qmax=127):
        check(self.lib.b200q_quantize_rows_with_range(self.handle, _ptr(y), M, N, ld_in, _ptr(row_min), _ptr(row_max), _ptr(q),
                                                      ld_out, _ptr(scales), qmin, qmax), "b200q_quantize_rows_with_range")

    def quantize_static(self, x, n, scale, zero_point, dst_kind, q):
        check(self.lib.b200q_quantize_static(self.handle, _ptr(x), n, scale, zero_point, dst_kind, _ptr(q)),
              "b200q_quantize_static")

    def dequantize_static(self, q, src_kind, n, scale, zero_point, y):
        check(self.lib.b200q_dequantize_static(self.handle, _ptr(q), src_kind, n, scale, zero_point, _ptr(y)),
              "b200q_dequantize_static")

    def quantize_weights_per_channel(self, w, N, K, layout, qw, scales32, scales64=None):
        check(self.lib.b200q_quantize_weights_per_channel(self.handle, _ptr(w), N, K, layout, _ptr(qw), _ptr(scales32),
                                                          _ptr(scales64)), "b200q_quantize_weights_per_channel")

    def transpose_i8(self, w_kn, K, N, w_nk):
        check(self.lib.b200q_transpose_i8(self.handle, _ptr(w_kn), K, N, _ptr(w_nk)), "b200q_transpose_i8")

    def int8_gemm_i32(self, A, W_nk, M, N, K, out, zpA=0, zpW=0):
        check(self.lib.b200q_int8_gemm_i32(self.handle, _ptr(A), _ptr(W_nk), M, N, K, zpA, zpW, _ptr(out)),
              "b200q_int8_gemm_i32")

    def epilogue(self, acc, M, N, a_scales, w_scales, bias, act, out):
        check(self.lib.b200q_epilogue(self.handle, _ptr(acc), M, N, _ptr(a_scales), _ptr(w_scales), _ptr(bias), ACT[act],
                                      _ptr(out)), "b200q_epilogue")

    def int8_linear(self, A, a_scales, W_nk, w_scales, bias, act, M, N, K, out):
        check(self.lib.b200q_int8_linear(self.handle, _ptr(A), _ptr(a_scales), _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act],
                                         M, N, K, _ptr(out)), "b200q_int8_linear")

    def int8_linear_requant_static(self, A, a_scales, W_nk, w_scales, bias, act, M, N, K, out_scale, out_q):
        check(self.lib.b200q_int8_linear_requant_static(self.handle, _ptr(A), _ptr(a_scales), _ptr(W_nk), _ptr(w_scales),
                                                        _ptr(bias), ACT[act], M, N, K, out_scale, _ptr(out_q)),
              "b200q_int8_linear_requant_static")

    def int8_linear_requant_token(self, A, a_scales, W_nk, w_scales, bias, act, M, N, K, out_q, out_scales):
        check(self.lib.b200q_int8_linear_requant_token(self.handle, _ptr(A), _ptr(a_scales), _ptr(W_nk), _ptr(w_scales),
                                                       _ptr(bias), ACT[act], M, N, K, _ptr(out_q), _ptr(out_scales)),
              "b200q_int8_linear_requant_token")

    def linear_f32(self, x, W_nk, w_scales, bias, act, M, N, K, out):
        check(self.lib.b200q_linear_f32(self.handle, _ptr(x), _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act], M, N, K,
                                        _ptr(out)), "b200q_linear_f32")

    def linear_f32_noalloc(self, x, W_nk, w_scales, bias, act, M, N, K, out):
        """b200q_linear_f32 without any allocation inside the call: scratch is a fixed array in the library
        (M*K <= 4 Mi, M <= 16384, tensor-core shapes only); overlapping calls on one GPU race on it."""
        check(self.lib.b200q_linear_f32_noalloc(self.handle, _ptr(x), _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act], M, N, K,
                                                _ptr(out)), "b200q_linear_f32_noalloc")

    # ---- ops (host buffers in and out; weights on the device)
    def linear_f32_host(self, x_host, W_nk, w_scales, bias, act, M, N, K, out_host):
        check(self.lib.b200q_linear_f32_host(self.handle, _ptr(x_host), _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act], M, N,
                                             K, _ptr(out_host)), "b200q_linear_f32_host")

    # ---- calibration observers
    def observer_reset(self, state):
        check(self.lib.b200q_observer_reset(self.handle, _ptr(state)), "b200q_observer_reset")

    def observe_minmax(self, x, n, state):
        check(self.lib.b200q_observe_minmax(self.handle, _ptr(x), n, _ptr(state)), "b200q_observe_minmax")

    # ---- f32 pieces of a transformer block
    def embedding_f32(self, table, tokens, pos_table, M, D, V, S, out):
        check(self.lib.b200q_embedding_f32(self.handle, _ptr(table), _ptr(tokens), _ptr(pos_table), M, D, V, S, _ptr(out)),
              "b200q_embedding_f32")

    def add_f32(self, a, b, n, out):
        check(self.lib.b200q_add_f32(self.handle, _ptr(a), _ptr(b), n, _ptr(out)), "b200q_add_f32")

    def layernorm_quantize(self, x, residual, gamma, beta, eps, M, D, sum_out=None, y_out=None, q_out=None, scales_out=None):
        check(self.lib.b200q_layernorm_quantize(self.handle, _ptr(x), _ptr(residual), _ptr(gamma), _ptr(beta), float(eps), M, D,
                                                _ptr(sum_out), _ptr(y_out), _ptr(q_out), _ptr(scales_out)),
              "b200q_layernorm_quantize")

    def set_sdpa_variant(self, variant: int):
        """0: CUDA-core binary32 FMA (default); 1: warp-level tensor-core instructions with three-way tf32 products."""
        check(self.lib.b200q_set_sdpa_variant(self.handle, variant), "b200q_set_sdpa_variant")

    def sdpa_f32(self, q, k, v, ld_q, ld_k, ld_v, B, H, S, head_dim, scale, causal, out, ld_out):
        check(self.lib.b200q_sdpa_f32(self.handle, _ptr(q), _ptr(k), _ptr(v), ld_q, ld_k, ld_v, B, H, S, head_dim, float(scale),
                                      int(bool(causal)), _ptr(out), ld_out), "b200q_sdpa_f32")

    def quant_roundtrip_host(self, x_host, M, K, q_host, scales_host, y_host):
        check(self.lib.b200q_quant_roundtrip_host(self.handle, _ptr(x_host), M, K, _ptr(q_host), _ptr(scales_host),
                                                  _ptr(y_host)), "b200q_quant_roundtrip_host")
