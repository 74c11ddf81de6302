"""Reader / writer of the reference's ``mlfw-ckpt-v1`` container, so that int8 weights, their scales and biases travel
in the same files as the rest of a model's state.

Format (src/lightning/io/checkpoint_format.ts:82-145 of the reference): an 8-byte little-endian header length, a
UTF-8 JSON header ``{"format": "mlfw-ckpt-v1", "tree": ..., "buffers": [...]}``, then the raw buffers back to back.
The tree mirrors the saved object; a tensor or typed array in it is ``{"$buf": index}``, a ``Map`` is
``{"$map": [[key, node], ...]}``.  Buffer metadata is ``{"kind": "tensor", "dtype", "shape", "offset", "length"}`` or
``{"kind": "array", "arrayType", "offset", "length"}`` with offsets relative to the first byte after the header.

Python side: a tensor is a :class:`TensorRecord` (dtype name of the reference + shape + numpy data), a typed array is
a 1-D numpy array, a ``Map`` is a :class:`collections.OrderedDict` (plain ``dict`` = plain object).
"""
from __future__ import annotations

import json
import struct
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, List, Tuple

import numpy as np

MAGIC = "mlfw-ckpt-v1"
HEADER_PREFIX_BYTES = 8

# dtype names of the reference (src/util/dtype_map.ts) <-> numpy; f16 / bf16 travel as their 16-bit patterns
DTYPE_TO_NUMPY = {"f32": np.float32, "f64": np.float64, "i8": np.int8, "ui8": np.uint8, "i16": np.int16, "i32": np.int32,
                  "i64": np.int64, "f16": np.uint16, "bf16": np.uint16, "bool": np.uint8}
ARRAY_TO_NUMPY = {"Int8Array": np.int8, "Uint8Array": np.uint8, "Uint8ClampedArray": np.uint8, "Int16Array": np.int16,
                  "Uint16Array": np.uint16, "Int32Array": np.int32, "Uint32Array": np.uint32, "Float32Array": np.float32,
                  "Float64Array": np.float64, "BigInt64Array": np.int64, "BigUint64Array": np.uint64}
NUMPY_TO_ARRAY = {np.dtype(v): k for k, v in ARRAY_TO_NUMPY.items() if k != "Uint8ClampedArray"}


@dataclass
class TensorRecord:
    """A ``Tensor`` of the reference: its dtype name, shape and contiguous data."""
    dtype: str
    shape: Tuple[int, ...]
    data: np.ndarray

    @staticmethod
    def of(array: np.ndarray, dtype: str = "") -> "TensorRecord":
        a = np.ascontiguousarray(array)
        if not dtype:
            dtype = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64", np.dtype(np.int8): "i8", np.dtype(np.uint8): "ui8",
                     np.dtype(np.int16): "i16", np.dtype(np.int32): "i32", np.dtype(np.int64): "i64"}[a.dtype]
        assert np.dtype(DTYPE_TO_NUMPY[dtype]) == a.dtype, f"{dtype} tensors hold {np.dtype(DTYPE_TO_NUMPY[dtype])} data"
        return TensorRecord(dtype, tuple(int(d) for d in a.shape), a)


def _encode(value: Any, buffers: List[Tuple[dict, bytes]]) -> Any:
    if isinstance(value, TensorRecord):
        buffers.append(({"kind": "tensor", "dtype": value.dtype, "shape": list(value.shape)},
                        np.ascontiguousarray(value.data).tobytes()))
        return {"$buf": len(buffers) - 1}
    if isinstance(value, np.ndarray):
        a = np.ascontiguousarray(value).reshape(-1)
        buffers.append(({"kind": "array", "arrayType": NUMPY_TO_ARRAY[a.dtype]}, a.tobytes()))
        return {"$buf": len(buffers) - 1}
    if isinstance(value, OrderedDict):
        return {"$map": [[k, _encode(v, buffers)] for k, v in value.items()]}
    if isinstance(value, (list, tuple)):
        return [_encode(v, buffers) for v in value]
    if isinstance(value, dict):
        return {str(k): _encode(v, buffers) for k, v in value.items()}
    if isinstance(value, (np.integer, np.floating, np.bool_)):
        value = value.item()
    if isinstance(value, float) and (value != value or value in (float("inf"), float("-inf"))):
        return None    # JSON.stringify writes null for NaN and the infinities; a bare NaN token would not parse there
    return value   # None, str, int, float, bool


def serialize_checkpoint(checkpoint: Any) -> bytes:
    buffers: List[Tuple[dict, bytes]] = []
    tree = _encode(checkpoint, buffers)
    offset = 0
    for meta, raw in buffers:
        meta["offset"] = offset
        meta["length"] = len(raw)
        offset += len(raw)
    # JSON.stringify writes no whitespace and keeps insertion order
    header = json.dumps({"format": MAGIC, "tree": tree, "buffers": [m for m, _ in buffers]}, separators=(",", ":"),
                        ensure_ascii=False, allow_nan=False).encode("utf-8")
    return struct.pack("<Q", len(header)) + header + b"".join(raw for _, raw in buffers)


def _decode(node: Any, decoded: list) -> Any:
    if node is None or not isinstance(node, (dict, list)):
        return node
    if isinstance(node, list):
        return [_decode(n, decoded) for n in node]
    if "$buf" in node and isinstance(node["$buf"], int):
        return decoded[node["$buf"]]
    if "$map" in node and isinstance(node["$map"], list):
        return OrderedDict((k, _decode(v, decoded)) for k, v in node["$map"])
    return {k: _decode(v, decoded) for k, v in node.items()}


def deserialize_checkpoint(blob: bytes) -> Any:
    (header_len,) = struct.unpack_from("<Q", blob, 0)
    start = HEADER_PREFIX_BYTES + header_len
    header = json.loads(blob[HEADER_PREFIX_BYTES:start].decode("utf-8"))
    if header.get("format") != MAGIC:
        raise ValueError("mlfw: unrecognized checkpoint format: " + str(header.get("format")))
    decoded = []
    for meta in header["buffers"]:
        raw = blob[start + meta["offset"]: start + meta["offset"] + meta["length"]]
        if meta["kind"] == "tensor":
            a = np.frombuffer(raw, dtype=DTYPE_TO_NUMPY[meta["dtype"]]).copy().reshape(meta["shape"])
            decoded.append(TensorRecord(meta["dtype"], tuple(meta["shape"]), a))
        else:
            if meta["arrayType"] not in ARRAY_TO_NUMPY:
                raise ValueError("mlfw: unknown typed array in checkpoint: " + str(meta["arrayType"]))
            decoded.append(np.frombuffer(raw, dtype=ARRAY_TO_NUMPY[meta["arrayType"]]).copy())
    return _decode(header["tree"], decoded)


def quantized_linear_state(weight_q: np.ndarray, scales: np.ndarray, bias=None) -> OrderedDict:
    """State of one int8 linear as it goes into a checkpoint's ``modelState`` map: the [N, K] int8 weight as an ``i8``
    tensor, its per-channel scales and the bias as ``f32`` tensors."""
    st = OrderedDict()
    st["weight_q"] = TensorRecord.of(np.ascontiguousarray(weight_q, np.int8))
    st["weight_scale"] = TensorRecord.of(np.ascontiguousarray(scales, np.float32))
    if bias is not None:
        st["bias"] = TensorRecord.of(np.ascontiguousarray(bias, np.float32))
    return st
