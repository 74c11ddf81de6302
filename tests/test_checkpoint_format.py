"""The ``mlfw-ckpt-v1`` container: byte layout against a hand-built known answer, and the reference's own round-trip
cases (tests/lightning/callbacks/checkpoint.test.js:19-55 of the reference) restated."""
import json
import struct
from collections import OrderedDict

import numpy as np
import pytest

from mlfw_b200.checkpoint import (TensorRecord, deserialize_checkpoint, quantized_linear_state, serialize_checkpoint)


def test_byte_layout_known_answer():
    """{"a": Int8Array [1,-2,3], "t": i8 tensor [[4,5]]} laid out by hand from checkpoint_format.ts:82-105."""
    blob = serialize_checkpoint({"a": np.array([1, -2, 3], np.int8), "t": TensorRecord.of(np.array([[4, 5]], np.int8))})
    header = ('{"format":"mlfw-ckpt-v1","tree":{"a":{"$buf":0},"t":{"$buf":1}},"buffers":['
              '{"kind":"array","arrayType":"Int8Array","offset":0,"length":3},'
              '{"kind":"tensor","dtype":"i8","shape":[1,2],"offset":3,"length":2}]}').encode()
    assert blob == struct.pack("<Q", len(header)) + header + bytes([1, 0xFE, 3, 4, 5])


def test_round_trips_tensors_exactly():
    w = TensorRecord.of(np.array([[1.5, -2.25], [3.125, np.pi]], np.float32))
    ids = TensorRecord.of(np.array([7, 8, 9], np.int32))
    ckpt = {"epoch": 3, "globalStep": 42, "modelState": OrderedDict([("w", w), ("ids", ids)])}
    back = deserialize_checkpoint(serialize_checkpoint(ckpt))
    assert back["epoch"] == 3 and back["globalStep"] == 42 and isinstance(back["modelState"], OrderedDict)
    rw, rids = back["modelState"]["w"], back["modelState"]["ids"]
    assert rw.shape == (2, 2) and rw.dtype == "f32" and (rw.data.view(np.uint32) == w.data.view(np.uint32)).all()
    assert rids.dtype == "i32" and rids.data.tolist() == [7, 8, 9]


def test_round_trips_optimizer_state():
    ckpt = {"optimizerStates": [{"paramGroups": [{"lr": 0.05, "betas": [0.9, 0.999]}],
                                 "state": OrderedDict([(0, {"step": 5, "exp_avg": np.array([0.1, 0.2, 0.3], np.float32)})])}]}
    back = deserialize_checkpoint(serialize_checkpoint(ckpt))
    opt = back["optimizerStates"][0]
    assert opt["paramGroups"][0] == {"lr": 0.05, "betas": [0.9, 0.999]}
    s = opt["state"][0]
    assert s["step"] == 5 and s["exp_avg"].dtype == np.float32
    assert s["exp_avg"].tolist() == [0.10000000149011612, 0.20000000298023224, 0.30000001192092896]


def test_payload_is_binary_not_text():
    big = TensorRecord.of((np.arange(4096) * 0.5).astype(np.float32))
    assert len(serialize_checkpoint({"modelState": OrderedDict([("w", big)])})) < 4096 * 4 * 1.4


def test_quantized_linear_state_round_trip():
    rng = np.random.default_rng(0)
    wq = rng.integers(-127, 128, size=(16, 32)).astype(np.int8)
    sc = rng.uniform(1e-3, 1e-2, 16).astype(np.float32)
    b = rng.standard_normal(16).astype(np.float32)
    ckpt = {"modelState": OrderedDict([("fc1", quantized_linear_state(wq, sc, b)), ("fc2", quantized_linear_state(wq.T.copy(), sc[:8].repeat(4)))])}
    blob = serialize_checkpoint(ckpt)
    (hl,) = struct.unpack_from("<Q", blob, 0)
    header = json.loads(blob[8:8 + hl])
    assert header["format"] == "mlfw-ckpt-v1" and [m["dtype"] for m in header["buffers"]] == ["i8", "f32", "f32", "i8", "f32"]
    assert header["buffers"][0]["shape"] == [16, 32] and header["buffers"][0]["length"] == 512
    back = deserialize_checkpoint(blob)["modelState"]
    assert (back["fc1"]["weight_q"].data == wq).all() and back["fc1"]["weight_q"].dtype == "i8"
    assert (back["fc1"]["weight_scale"].data.view(np.uint32) == sc.view(np.uint32)).all()
    assert (back["fc1"]["bias"].data == b).all() and "bias" not in back["fc2"]


def test_rejects_other_formats():
    bad = b'{"format":"other","tree":null,"buffers":[]}'
    with pytest.raises(ValueError):
        deserialize_checkpoint(struct.pack("<Q", len(bad)) + bad)
