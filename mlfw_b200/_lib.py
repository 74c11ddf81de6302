"""ctypes binding of ``libb200q.so`` — one prototype per declaration in ``include/b200q.h``.

There is no fallback: if the library is missing or fails to load the import of the
package raises, and every call that returns non-zero raises :class:`B200QError`
with the library's own message.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200q.so")

c_i64, c_int, c_dbl, c_vp, c_sz = C.c_int64, C.c_int, C.c_double, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); kept in the order of the header
PROTOTYPES = {
    "b200q_device_count": (c_int, []),
    "b200q_create": (c_int, [c_int, C.POINTER(c_vp)]),
    "b200q_destroy": (None, [c_vp]),
    "b200q_last_error": (C.c_char_p, []),
    "b200q_sync": (c_int, [c_vp]),
    "b200q_status_word": (c_int, [c_vp, C.POINTER(C.c_uint32)]),
    "b200q_clear_status": (c_int, [c_vp]),
    "b200q_set_wait_limit": (c_int, [c_vp, c_dbl]),
    "b200q_set_gemm_variant": (c_int, [c_vp, c_int]),
    "b200q_set_tail_mode": (c_int, [c_vp, c_int]),
    "b200q_set_epilogue_warps": (c_int, [c_vp, c_int]),
    "b200q_set_host_threads": (c_int, [c_vp, c_int]),
    "b200q_set_tile_group": (c_int, [c_vp, c_int]),
    "b200q_set_requant_variant": (c_int, [c_vp, c_int]),
    "b200q_set_quant_variant": (c_int, [c_vp, c_int]),
    "b200q_launch_count": (C.c_uint64, [c_vp]),
    "b200q_sm_count": (c_int, [c_vp]),
    "b200q_alloc": (c_int, [c_vp, c_sz, C.POINTER(c_vp)]),
    "b200q_free": (c_int, [c_vp, c_vp]),
    "b200q_memset": (c_int, [c_vp, c_vp, c_int, c_sz]),
    "b200q_upload": (c_int, [c_vp, c_vp, c_vp, c_sz]),
    "b200q_download": (c_int, [c_vp, c_vp, c_vp, c_sz]),
    "b200q_host_alloc": (c_int, [c_vp, c_sz, C.POINTER(c_vp)]),
    "b200q_host_free": (c_int, [c_vp, c_vp]),
    "b200q_host_register": (c_int, [c_vp, c_vp, c_sz]),
    "b200q_host_unregister": (c_int, [c_vp, c_vp]),
    "b200q_timer_start": (c_int, [c_vp]),
    "b200q_timer_stop": (c_int, [c_vp, C.POINTER(C.c_float)]),
    "b200q_profile_enable": (c_int, [c_vp, c_int]),
    "b200q_profile_reset": (c_int, [c_vp]),
    "b200q_profile_read": (c_int, [c_vp, c_int, C.POINTER(c_dbl), C.POINTER(C.c_uint64)]),
    "b200q_quantize_per_token": (c_int, [c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_int, c_int]),
    "b200q_dequantize_per_token": (c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_vp]),
    "b200q_row_range": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "b200q_quantize_rows_with_range": (c_int, [c_vp, c_vp, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp, c_i64, c_vp, c_int, c_int]),
    "b200q_quantize_static": (c_int, [c_vp, c_vp, c_i64, c_dbl, c_int, c_int, c_vp]),
    "b200q_dequantize_static": (c_int, [c_vp, c_vp, c_int, c_i64, c_dbl, c_int, c_vp]),
    "b200q_quantize_weights_per_channel": (c_int, [c_vp, c_vp, c_i64, c_i64, c_int, c_vp, c_vp, c_vp]),
    "b200q_transpose_i8": (c_int, [c_vp, c_vp, c_i64, c_i64, c_vp]),
    "b200q_quantize_per_group": (c_int, [c_vp, c_vp, c_i64, c_i64, c_int, c_vp, c_vp, c_vp]),
    "b200q_dequantize_per_group": (c_int, [c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "b200q_quantized_conv2d": (c_int, [c_vp, c_vp, c_vp] + [c_i64] * 7 + [c_int] * 12 + [c_vp]),
    "b200q_shift_u8_to_i8": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "b200q_int8_gemm_i32": (c_int, [c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_int, c_int, c_vp]),
    "b200q_epilogue": (c_int, [c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp, c_int, c_vp]),
    "b200q_epilogue_tensor_scale": (c_int, [c_vp, c_vp, c_i64, c_i64, C.c_double, c_vp, c_int, c_vp]),
    "b200q_int8_linear": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "b200q_int8_linear_gathered": (c_int, [c_vp, c_vp, c_vp, c_int, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "b200q_int8_linear_requant_static": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_dbl, c_vp]),
    "b200q_int8_linear_requant_token": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp, c_vp]),
    "b200q_int8_linear_f32_requant_token": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "b200q_linear_f32": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "b200q_linear_f32_noalloc": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "b200q_linear_f32_host": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "b200q_linear_f32_many": (c_int, [c_vp, c_int, c_vp, c_vp, c_vp, c_vp, c_int, c_i64, c_i64, c_i64, c_vp]),
    "b200q_quant_roundtrip_host": (c_int, [c_vp, c_vp, c_i64, c_i64, c_vp, c_vp, c_vp]),
    "b200q_observer_reset": (c_int, [c_vp, c_vp]),
    "b200q_observe_minmax": (c_int, [c_vp, c_vp, c_i64, c_vp]),
    "b200q_histogram_f32": (c_int, [c_vp, c_vp, c_i64, c_dbl, c_dbl, c_int, c_vp]),
    "b200q_histogram_percentile_threshold": (c_int, [c_vp, c_int, c_dbl, c_dbl, c_dbl, c_dbl, C.POINTER(c_dbl)]),
    "b200q_histogram_entropy_threshold": (c_int, [c_vp, c_int, c_dbl, c_dbl, c_dbl, c_int, C.POINTER(c_dbl)]),
    "b200q_embedding_f32": (c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_vp]),
    "b200q_add_f32": (c_int, [c_vp, c_vp, c_vp, c_i64, c_vp]),
    "b200q_layernorm_quantize": (c_int, [c_vp, c_vp, c_vp, c_vp, c_vp, C.c_float, c_i64, c_i64, c_vp, c_vp, c_vp, c_vp]),
    "b200q_set_sdpa_variant": (c_int, [c_vp, c_int]),
    "b200q_sdpa_f32": (c_int, [c_vp, c_vp, c_vp, c_vp, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, c_i64, C.c_float, c_int, c_vp, c_i64]),
    "b200q_graph_begin": (c_int, [c_vp]),
    "b200q_graph_end": (c_int, [c_vp, C.POINTER(c_vp)]),
    "b200q_graph_launch": (c_int, [c_vp, c_vp]),
    "b200q_graph_destroy": (c_int, [c_vp, c_vp]),
    "b200q_selftest_bounded_wait": (c_int, [c_vp, c_dbl]),
    "b200q_group_unique_id": (c_int, [c_vp]),
    "b200q_group_create": (c_int, [C.POINTER(c_int), c_int, C.POINTER(c_vp)]),
    "b200q_group_create_rank": (c_int, [c_vp, c_vp, c_int, c_int, C.POINTER(c_vp)]),
    "b200q_group_destroy": (c_int, [c_vp]),
    "b200q_group_world": (c_int, [c_vp]),
    "b200q_group_local_count": (c_int, [c_vp]),
    "b200q_group_ctx": (c_vp, [c_vp, c_int]),
    "b200q_group_rank": (c_int, [c_vp, c_int]),
    "b200q_group_nccl_version": (c_int, [c_vp, C.POINTER(c_int)]),
    "b200q_group_sync": (c_int, [c_vp]),
    "b200q_group_linear_mshard": (c_int, [c_vp, C.POINTER(c_vp), C.POINTER(c_i64), C.POINTER(c_vp), C.POINTER(c_vp), C.POINTER(c_vp),
                                          c_int, c_i64, c_i64, C.POINTER(c_vp)]),
    "b200q_group_linear_nshard": (c_int, [c_vp, C.POINTER(c_vp), C.POINTER(c_vp), c_int, C.POINTER(c_vp), C.POINTER(c_vp),
                                          C.POINTER(c_vp), c_int, c_i64, c_i64, c_i64, C.POINTER(c_vp), C.POINTER(c_vp), C.POINTER(c_vp)]),
    "b200q_group_set_chunks": (c_int, [c_vp, c_int]),
    "b200q_group_fence": (c_int, [c_vp]),
    "b200q_group_all_gather": (c_int, [c_vp, C.POINTER(c_vp), C.POINTER(c_vp), c_sz]),
}


class B200QError(RuntimeError):
    pass


def load(path: str = LIB_PATH) -> C.CDLL:
    if not os.path.exists(path):
        raise B200QError(f"{path} is missing: build it with `python -m mlfw_b200.build` (nvcc, sm_100a). "
                         "This backend has no CPU fallback.")
    lib = C.CDLL(path)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError here means the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


_LIB = None


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = load()
    return _LIB


def check(code: int, what: str = "") -> None:
    if code != 0:
        msg = lib().b200q_last_error()
        raise B200QError(f"{what}: {msg.decode() if msg else 'error'} (code {code})")
