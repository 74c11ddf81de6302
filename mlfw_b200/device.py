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
               8: "unexpected tensor-memory allocation", 16: "staged quantize wait ran out", 32: "embedding index outside its table",
               64: "self test: the wait on a barrier nothing signals gave up (as it must)", 128: "attention kernel's wait for its MMAs ran out"}


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

    def __init__(self, device: int = 0, _borrowed_handle=None):
        self.lib = _lib.lib()
        self.device = device
        self._owned = _borrowed_handle is None
        if _borrowed_handle is not None:      # a context that belongs to a Group
            self.handle = _borrowed_handle
            return
        h = C.c_void_p()
        check(self.lib.b200q_create(device, C.byref(h)), "b200q_create")
        self.handle = h.value

    def close(self):
        if self.handle and self._owned:
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

    def host_register(self, arr: np.ndarray) -> None:
        """Page-locks a contiguous numpy array in place (b200q_host_register): the host-buffer calls then copy from / to it
        directly.  Call :meth:`host_unregister` before the array goes away."""
        assert arr.flags["C_CONTIGUOUS"] and arr.nbytes > 0
        check(self.lib.b200q_host_register(self.handle, arr.ctypes.data, arr.nbytes), "b200q_host_register")

    def host_unregister(self, arr: np.ndarray) -> None:
        check(self.lib.b200q_host_unregister(self.handle, arr.ctypes.data), "b200q_host_unregister")

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

    def set_tile_group(self, row_blocks: int):
        """Tile walking order of the tensor-core GEMM: -1 by size, 0 row block by row block, g groups of g row blocks."""
        check(self.lib.b200q_set_tile_group(self.handle, row_blocks), "b200q_set_tile_group")

    def set_host_threads(self, threads: int):
        """Host threads that stage pageable arrays of the host-buffer entry points (0: half the cores, at most 8)."""
        check(self.lib.b200q_set_host_threads(self.handle, threads), "b200q_set_host_threads")

    def set_epilogue_warps(self, warps: int):
        """Epilogue warps of the tensor-core GEMM for f32 output: 0 = sixteen for K <= 1024, eight otherwise (default); 8; 16."""
        check(self.lib.b200q_set_epilogue_warps(self.handle, warps), "b200q_set_epilogue_warps")

    def set_requant_variant(self, variant: int):
        """0: row ranges out of the GEMM epilogue + one-pass encode (default); 1: full per-token quantize of the f32 result."""
        check(self.lib.b200q_set_requant_variant(self.handle, variant), "b200q_set_requant_variant")

    def selftest_bounded_wait(self, limit_seconds: float):
        check(self.lib.b200q_selftest_bounded_wait(self.handle, limit_seconds), "b200q_selftest_bounded_wait")

    # ---- captured steps
    def graph_begin(self):
        check(self.lib.b200q_graph_begin(self.handle), "b200q_graph_begin")

    def graph_end(self) -> int:
        g = C.c_void_p()
        check(self.lib.b200q_graph_end(self.handle, C.byref(g)), "b200q_graph_end")
        return g.value

    def graph_launch(self, graph: int):
        check(self.lib.b200q_graph_launch(self.handle, graph), "b200q_graph_launch")

    def graph_destroy(self, graph: int):
        check(self.lib.b200q_graph_destroy(self.handle, graph), "b200q_graph_destroy")

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

    def quantize_per_group(self, x, n, group_size, num_bits, q, scales64=None, scales32=None):
        """Per-group (INT4-style) scales and codes of the flat f32 array x[n]; one code per int8."""
        check(self.lib.b200q_quantize_per_group(self.handle, _ptr(x), n, group_size, num_bits, _ptr(q), _ptr(scales64),
                                                _ptr(scales32)), "b200q_quantize_per_group")

    def dequantize_per_group(self, q, n, group_size, scales64, y64=None, y32=None):
        check(self.lib.b200q_dequantize_per_group(self.handle, _ptr(q), n, group_size, _ptr(scales64), _ptr(y64), _ptr(y32)),
              "b200q_dequantize_per_group")

    def quantized_conv2d(self, x, ker, shape, kernel_shape, out, strides=(1, 1), padding=((0, 0), (0, 0)), dilation=(1, 1),
                         groups=1, zp_in=0, zp_ker=0, layout="NCHW"):
        """quantized_conv: ``shape`` = (N, C, H, W) and ``kernel_shape`` = (O, KH, KW) whatever the layout
        ("NCHW" with an OIHW kernel, or "NHWC" with an OHWI kernel); int32 output in the input's layout."""
        N, Cc, H, W = shape
        O, KH, KW = kernel_shape
        check(self.lib.b200q_quantized_conv2d(self.handle, _ptr(x), _ptr(ker), N, Cc, H, W, O, KH, KW, strides[0], strides[1],
                                              padding[0][0], padding[0][1], padding[1][0], padding[1][1], dilation[0], dilation[1],
                                              groups, zp_in, zp_ker, {"NCHW": 0, "NHWC": 1}[layout], _ptr(out)),
              "b200q_quantized_conv2d")

    def transpose_i8(self, w_kn, K, N, w_nk):
        check(self.lib.b200q_transpose_i8(self.handle, _ptr(w_kn), K, N, _ptr(w_nk)), "b200q_transpose_i8")

    def shift_u8_to_i8(self, src, n, dst):
        """dst = src - 128 as int8 (ui8 operands of the contractions: move the zero-point by 128 as well)."""
        check(self.lib.b200q_shift_u8_to_i8(self.handle, _ptr(src), n, _ptr(dst)), "b200q_shift_u8_to_i8")

    def int8_gemm_i32(self, A, W_nk, M, N, K, out, zpA=0, zpW=0):
        check(self.lib.b200q_int8_gemm_i32(self.handle, _ptr(A), _ptr(W_nk), M, N, K, zpA, zpW, _ptr(out)),
              "b200q_int8_gemm_i32")

    def epilogue(self, acc, M, N, a_scales, w_scales, bias, act, out):
        check(self.lib.b200q_epilogue(self.handle, _ptr(acc), M, N, _ptr(a_scales), _ptr(w_scales), _ptr(bias), ACT[act],
                                      _ptr(out)), "b200q_epilogue")

    def epilogue_tensor_scale(self, acc, M, N, scale, bias, act, out):
        """act(fround(fround((double)acc * scale) + bias)): the compiled per-tensor `dequantize` and what follows it."""
        check(self.lib.b200q_epilogue_tensor_scale(self.handle, _ptr(acc), M, N, float(scale), _ptr(bias), ACT[act], _ptr(out)),
              "b200q_epilogue_tensor_scale")

    def int8_linear(self, A, a_scales, W_nk, w_scales, bias, act, M, N, K, out):
        check(self.lib.b200q_int8_linear(self.handle, _ptr(A), _ptr(a_scales), _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act],
                                         M, N, K, _ptr(out)), "b200q_int8_linear")

    def int8_linear_gathered(self, A, a_scales, a_blocks, W_nk, w_scales, bias, act, M, N, K, out):
        """int8_linear with A stored as ``a_blocks`` column blocks (the layout an all-gather of column shards leaves)."""
        check(self.lib.b200q_int8_linear_gathered(self.handle, _ptr(A), _ptr(a_scales), a_blocks, _ptr(W_nk), _ptr(w_scales),
                                                  _ptr(bias), ACT[act], M, N, K, _ptr(out)), "b200q_int8_linear_gathered")

    def int8_linear_requant_static(self, A, a_scales, W_nk, w_scales, bias, act, M, N, K, out_scale, out_q):
        check(self.lib.b200q_int8_linear_requant_static(self.handle, _ptr(A), _ptr(a_scales), _ptr(W_nk), _ptr(w_scales),
                                                        _ptr(bias), ACT[act], M, N, K, out_scale, _ptr(out_q)),
              "b200q_int8_linear_requant_static")

    def int8_linear_requant_token(self, A, a_scales, W_nk, w_scales, bias, act, M, N, K, out_q, out_scales):
        check(self.lib.b200q_int8_linear_requant_token(self.handle, _ptr(A), _ptr(a_scales), _ptr(W_nk), _ptr(w_scales),
                                                       _ptr(bias), ACT[act], M, N, K, _ptr(out_q), _ptr(out_scales)),
              "b200q_int8_linear_requant_token")

    def int8_linear_f32_requant_token(self, A, a_scales, W_nk, w_scales, bias, act, M, N, K, out_f32, out_q, out_scales):
        check(self.lib.b200q_int8_linear_f32_requant_token(self.handle, _ptr(A), _ptr(a_scales), _ptr(W_nk), _ptr(w_scales),
                                                           _ptr(bias), ACT[act], M, N, K, _ptr(out_f32), _ptr(out_q), _ptr(out_scales)),
              "b200q_int8_linear_f32_requant_token")

    def linear_f32(self, x, W_nk, w_scales, bias, act, M, N, K, out):
        check(self.lib.b200q_linear_f32(self.handle, _ptr(x), _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act], M, N, K,
                                        _ptr(out)), "b200q_linear_f32")

    def linear_f32_noalloc(self, x, W_nk, w_scales, bias, act, M, N, K, out):
        """b200q_linear_f32 without any allocation inside the call: scratch is a fixed array in the library
        (M*K <= 4 Mi, M <= 16384, tensor-core shapes only); overlapping calls on one GPU race on it."""
        check(self.lib.b200q_linear_f32_noalloc(self.handle, _ptr(x), _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act], M, N, K,
                                                _ptr(out)), "b200q_linear_f32_noalloc")

    # ---- ops (host buffers in and out; weights on the device)
    def linear_f32_many(self, xs, W_nk, w_scales, bias, act, M, N, K, outs):
        """Independent batches through one linear: the quantize of batch i+1 overlaps the GEMM of batch i."""
        n = len(xs)
        if len(outs) != n:
            raise ValueError("one output per batch")
        px = (C.c_void_p * n)(*[_ptr(v) for v in xs])
        po = (C.c_void_p * n)(*[_ptr(v) for v in outs])
        check(self.lib.b200q_linear_f32_many(self.handle, n, px, _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act], M, N, K, po),
              "b200q_linear_f32_many")

    def linear_f32_host(self, x_host, W_nk, w_scales, bias, act, M, N, K, out_host):
        check(self.lib.b200q_linear_f32_host(self.handle, _ptr(x_host), _ptr(W_nk), _ptr(w_scales), _ptr(bias), ACT[act], M, N,
                                             K, _ptr(out_host)), "b200q_linear_f32_host")

    # ---- calibration observers
    def observer_reset(self, state):
        check(self.lib.b200q_observer_reset(self.handle, _ptr(state)), "b200q_observer_reset")

    def observe_minmax(self, x, n, state):
        check(self.lib.b200q_observe_minmax(self.handle, _ptr(x), n, _ptr(state)), "b200q_observe_minmax")

    def histogram_f32(self, x, n, range_min, range_max, num_bins, bins):
        check(self.lib.b200q_histogram_f32(self.handle, _ptr(x), n, float(range_min), float(range_max), num_bins, _ptr(bins)),
              "b200q_histogram_f32")

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
        """0: tcgen05 kernel with three-way tf32 products when the alignment allows (default); 1: warp-level mma.sync, three-way
        tf32; 2: tcgen05 or an error; 3: CUDA-core binary32 FMA."""
        check(self.lib.b200q_set_sdpa_variant(self.handle, variant), "b200q_set_sdpa_variant")

    def sdpa_f32(self, q, k, v, ld_q, ld_k, ld_v, B, H, S, head_dim, scale, causal, out, ld_out):
        check(self.lib.b200q_sdpa_f32(self.handle, _ptr(q), _ptr(k), _ptr(v), ld_q, ld_k, ld_v, B, H, S, head_dim, float(scale),
                                      int(bool(causal)), _ptr(out), ld_out), "b200q_sdpa_f32")

    def quant_roundtrip_host(self, x_host, M, K, q_host, scales_host, y_host):
        check(self.lib.b200q_quant_roundtrip_host(self.handle, _ptr(x_host), M, K, _ptr(q_host), _ptr(scales_host),
                                                  _ptr(y_host)), "b200q_quant_roundtrip_host")


def _preload_nccl():
    """The library takes the NCCL that is already in the process.  In a Python process that is, sooner or later, the
    one torch is built against (``nvidia.nccl`` in site-packages), and a second, different build next to it breaks
    torch's import: so that one is loaded first when it exists.  Without it the library finds the system's."""
    import importlib.util
    import os
    try:
        spec = importlib.util.find_spec("nvidia.nccl")
    except (ImportError, ValueError):
        spec = None
    for base in (spec.submodule_search_locations if spec is not None and spec.submodule_search_locations else []):
        path = os.path.join(base, "lib", "libnccl.so.2")
        if os.path.exists(path):
            C.CDLL(path, mode=C.RTLD_GLOBAL)
            return path
    return None


def _ptr_array(items):
    """ctypes array of device addresses (None entries become null)."""
    arr = (C.c_void_p * len(items))()
    for i, b in enumerate(items):
        arr[i] = _ptr(b)
    return arr


class Group:
    """Several GPUs of one node behind one NCCL communicator (``b200q_group_*``).

    ``Group(devices=[0, 1])``: this process drives every rank (the group owns one context per device).
    ``Group.join(ctx, unique_id, rank, world)``: one process per GPU; ``Group.unique_id()`` on one rank makes the id,
    the host distributes it.  Per-GPU arguments are lists with one entry per local rank."""

    def __init__(self, devices=None, _handle=None, _contexts=None):
        self.lib = _lib.lib()
        _preload_nccl()
        if _handle is not None:
            self.handle, self.contexts = _handle, _contexts
            return
        devs = (C.c_int * len(devices))(*devices)
        h = C.c_void_p()
        check(self.lib.b200q_group_create(devs, len(devices), C.byref(h)), "b200q_group_create")
        self.handle = h.value
        self.contexts = [Context(d, _borrowed_handle=self.lib.b200q_group_ctx(self.handle, i)) for i, d in enumerate(devices)]

    @staticmethod
    def unique_id() -> bytes:
        _preload_nccl()
        buf = C.create_string_buffer(128)
        check(_lib.lib().b200q_group_unique_id(buf), "b200q_group_unique_id")
        return buf.raw

    @classmethod
    def join(cls, ctx: Context, unique_id: bytes, rank: int, world: int) -> "Group":
        assert len(unique_id) == 128
        _preload_nccl()
        h = C.c_void_p()
        buf = C.create_string_buffer(unique_id, 128)
        check(ctx.lib.b200q_group_create_rank(ctx.handle, buf, rank, world, C.byref(h)), "b200q_group_create_rank")
        return cls(_handle=h.value, _contexts=[ctx])

    def close(self):
        if self.handle:
            for c in self.contexts:
                if not c._owned:
                    c.handle = None
            check(self.lib.b200q_group_destroy(self.handle), "b200q_group_destroy")
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def world(self) -> int:
        return self.lib.b200q_group_world(self.handle)

    @property
    def local_count(self) -> int:
        return self.lib.b200q_group_local_count(self.handle)

    def rank(self, local_index: int = 0) -> int:
        return self.lib.b200q_group_rank(self.handle, local_index)

    def nccl_version(self) -> int:
        v = C.c_int()
        check(self.lib.b200q_group_nccl_version(self.handle, C.byref(v)), "b200q_group_nccl_version")
        return v.value

    def sync(self):
        check(self.lib.b200q_group_sync(self.handle), "b200q_group_sync")

    def fence(self):
        check(self.lib.b200q_group_fence(self.handle), "b200q_group_fence")

    def set_chunks(self, chunks: int):
        check(self.lib.b200q_group_set_chunks(self.handle, chunks), "b200q_group_set_chunks")

    def linear_mshard(self, x, rows, W_nk, w_scales, bias, act, N, K, out):
        r = (C.c_int64 * len(rows))(*rows)
        check(self.lib.b200q_group_linear_mshard(self.handle, _ptr_array(x), r, _ptr_array(W_nk), _ptr_array(w_scales),
                                                 _ptr_array(bias) if bias is not None else None, ACT[act], N, K, _ptr_array(out)),
              "b200q_group_linear_mshard")

    def linear_nshard(self, q_in, in_scales, in_blocks, W_shard, w_scales, bias, act, M, N, K, q_out=None, out_scales=None, out_f32=None):
        check(self.lib.b200q_group_linear_nshard(self.handle, _ptr_array(q_in), _ptr_array(in_scales), in_blocks, _ptr_array(W_shard),
                                                 _ptr_array(w_scales), _ptr_array(bias) if bias is not None else None, ACT[act], M, N, K,
                                                 _ptr_array(q_out) if q_out is not None else None,
                                                 _ptr_array(out_scales) if out_scales is not None else None,
                                                 _ptr_array(out_f32) if out_f32 is not None else None), "b200q_group_linear_nshard")

    def all_gather(self, send, recv, nbytes: int):
        check(self.lib.b200q_group_all_gather(self.handle, _ptr_array(send), _ptr_array(recv), nbytes), "b200q_group_all_gather")
