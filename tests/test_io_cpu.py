"""`save` / `load`: the byte layout of the reference's checkpoint format, version 1
(python/quabla/_io.py:1-35), round trips, and refusal of malformed files."""

import io
import json
import math
import struct

import numpy as np
import pytest

import quabla_b200 as qb

MAGIC = b"\x93QUABLA\n"


def _file(header: dict, data: bytes = b"") -> bytes:
    text = json.dumps(header, separators=(",", ":")).encode()
    return MAGIC + struct.pack("<Q", len(text)) + text + data


def _saved(tree) -> bytes:
    buffer = io.BytesIO()
    qb.save(buffer, tree)
    return buffer.getvalue()


def test_layout_is_the_documented_one_byte_for_byte():
    w = np.array([[1.0, -2.0, 0.5]], dtype=np.float32)
    mask = np.array([True, False])
    tree = {"step": 3, "rate": 1.5, "name": "tanh", "w": w, 7: (None, mask), "flags": [True]}
    header = {
        "format": "quabla", "version": 1,
        "tree": {"type": "dict", "keys": ["step", "rate", "name", "w", 7, "flags"], "values": [
            {"type": "int", "value": 3},
            {"type": "float", "value": "0x1.8000000000000p+0"},
            {"type": "str", "value": "tanh"},
            {"type": "array", "dtype": "float32", "shape": [1, 3], "offset": 0, "nbytes": 12},
            {"type": "tuple", "items": [{"type": "none"},
                                        {"type": "array", "dtype": "bool", "shape": [2], "offset": 12, "nbytes": 2}]},
            {"type": "list", "items": [{"type": "bool", "value": True}]},
        ]},
    }
    data = struct.pack("<3f", 1.0, -2.0, 0.5) + b"\x01\x00"
    assert _saved(tree) == _file(header, data)


def test_round_trip_keeps_types_bits_and_key_order(tmp_path):
    rng = np.random.default_rng(5)
    tree = {"b": [rng.standard_normal((3, 4)), rng.standard_normal(5).astype(np.float32)],
            "a": ({"z": np.zeros((0, 2)), 1: np.float64(2.5)}, None, -0.0, math.inf, 5e-324, 2**70, "π", False),
            "scalar": np.array(3.25, dtype=np.float32)}
    path = tmp_path / "state.qb"
    qb.save(path, tree)
    back = qb.load(path)
    assert list(back) == ["b", "a", "scalar"] and list(back["a"][0]) == ["z", 1]
    assert type(back["a"]) is tuple and type(back["b"]) is list
    for got, want in zip(back["b"], tree["b"]):
        assert got.dtype == want.dtype and got.shape == want.shape and got.tobytes() == want.tobytes()
    assert back["a"][0]["z"].shape == (0, 2)
    assert back["a"][0][1].shape == () and back["a"][0][1] == 2.5  # a NumPy scalar is saved as a 0-d array
    assert back["a"][1] is None and math.copysign(1.0, back["a"][2]) == -1.0
    assert back["a"][3:] == (math.inf, 5e-324, 2**70, "π", False) and type(back["a"][7]) is bool
    assert back["scalar"].dtype == np.float32 and back["scalar"].shape == ()
    assert back["b"][0].flags.writeable and back["b"][0].flags.aligned
    # A non-contiguous view is written in C order.
    view = np.arange(12.0).reshape(3, 4).T
    assert np.array_equal(qb.load(io.BytesIO(_saved(view))), view)


def test_big_endian_input_is_written_little_endian():
    value = np.arange(4, dtype=">f8")
    assert _saved(value)[-32:] == np.arange(4, dtype="<f8").tobytes()


@pytest.mark.parametrize("leaf", [np.arange(3), np.zeros(2, dtype=np.float16), {1.5: 0}, {(1, 2): 0}, object(), {1, 2},
                                  np.zeros(2, dtype=np.complex128), b"bytes"])
def test_unsupported_leaves_are_refused(leaf):
    with pytest.raises(TypeError):
        _saved({"x": leaf} if not isinstance(leaf, dict) else leaf)


def test_nan_floats_are_saved_exactly_as_hex():
    back = qb.load(io.BytesIO(_saved([math.nan, -math.inf])))
    assert math.isnan(back[0]) and back[1] == -math.inf


NAN_HEADER = b'{"format":"quabla","version":1,"tree":{"type":"list","items":[NaN]}}'


def _array_node(**changes):
    node = {"type": "array", "dtype": "float64", "shape": [2], "offset": 0, "nbytes": 16}
    node.update(changes)
    return {"format": "quabla", "version": 1, "tree": node}


@pytest.mark.parametrize("content", [
    b"", b"\x93NUMPY\n" + bytes(20), MAGIC, MAGIC + struct.pack("<Q", 50) + b"{}",
    MAGIC + struct.pack("<Q", 4) + b"\xff\xfe{}", MAGIC + struct.pack("<Q", 2) + b"{]",
    _file({"format": "other", "version": 1, "tree": {"type": "none"}}),
    _file({"format": "quabla", "version": 2, "tree": {"type": "none"}}),
    _file({"format": "quabla", "version": True, "tree": {"type": "none"}}),
    _file({"format": "quabla", "version": 1}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "set"}}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "int", "value": True}}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "bool", "value": 1}}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "float", "value": 1.5}}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "float", "value": "one"}}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "list", "items": {"0": 1}}}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "dict", "keys": ["a", "a"],
                                                       "values": [{"type": "none"}, {"type": "none"}]}}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "dict", "keys": ["a"], "values": []}}),
    _file({"format": "quabla", "version": 1, "tree": {"type": "dict", "keys": [1.5], "values": [{"type": "none"}]}}),
    _file(_array_node(), bytes(15)),                      # data section too short
    _file(_array_node(nbytes=8), bytes(16)),              # byte count does not match the shape
    _file(_array_node(dtype="int32"), bytes(16)),
    _file(_array_node(shape=[-2]), bytes(16)),
    _file(_array_node(shape=[2.0]), bytes(16)),
    _file(_array_node(offset=-8), bytes(16)),
    _file(_array_node(offset=8), bytes(16)),
    _file(_array_node(dtype="bool", nbytes=2), b"\x01\x02"),  # bool bytes must be 0 or 1
    MAGIC + struct.pack("<Q", len(NAN_HEADER)) + NAN_HEADER,  # JSON has no NaN token
])
def test_malformed_files_raise_value_error(content):
    with pytest.raises(ValueError):
        qb.load(io.BytesIO(content))


def test_deep_nesting_is_a_value_error_not_a_crash():
    text = b'{"format":"quabla","version":1,"tree":' + b'{"type":"list","items":[' * 100000 + b'{"type":"none"}' + b"]}" * 100000 + b"}"
    with pytest.raises(ValueError):
        qb.load(io.BytesIO(MAGIC + struct.pack("<Q", len(text)) + text))


def test_a_stream_that_stalls_is_an_os_error():
    class Stalled:
        def write(self, data):
            return 0

    with pytest.raises(OSError):
        qb.save(Stalled(), [1.0])
