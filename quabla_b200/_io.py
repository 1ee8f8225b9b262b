"""`save` / `load` of pytrees of arrays in the reference's checkpoint file format, version 1
(python/quabla/_io.py:1-35 documents the layout; files are interchangeable with the reference's
`quabla.save` / `quabla.load`, byte for byte for the same tree).

    offset 0     8 bytes   b"\\x93QUABLA\\n"
    offset 8     8 bytes   N, unsigned little-endian
    offset 16    N bytes   UTF-8 JSON, compact separators, no NaN/Infinity tokens:
                           {"format":"quabla","version":1,"tree":NODE}
    offset 16+N            array bytes, concatenated in tree order

NODE is {"type":"none"} | {"type":"bool"|"int"|"str","value":v} | {"type":"float","value":float.hex}
| {"type":"list"|"tuple","items":[NODE…]} | {"type":"dict","keys":[str or int…],"values":[NODE…]}
| {"type":"array","dtype":"float64"|"float32"|"bool","shape":[…],"offset":o,"nbytes":n}, with `o`
relative to the data section; arrays are C-ordered little-endian, bool one byte (0 or 1) per element.

Arrays are NumPy arrays here (the host-side array type of this package); NumPy scalars are saved
as zero-dimensional arrays.  Loading never unpickles or imports anything named by the file, and
every malformed or truncated file raises `ValueError`.
"""

from __future__ import annotations

import json
import os
import struct
from typing import Any

import numpy as np

__all__ = ["save", "load"]

MAGIC = b"\x93QUABLA\n"
VERSION = 1
_SIZE = struct.Struct("<Q")
_ARRAY_TYPES = {"float64": np.dtype("<f8"), "float32": np.dtype("<f4"), "bool": np.dtype(np.bool_)}


class _Writer:
    """Builds the header tree and collects the array bytes in tree order."""

    def __init__(self) -> None:
        self.blobs: list[bytes] = []
        self.cursor = 0

    def node(self, value: Any) -> dict:
        if value is None:
            return {"type": "none"}
        kind = type(value)
        if kind in (bool, int, str):
            return {"type": kind.__name__, "value": value}
        if kind is float:
            return {"type": "float", "value": value.hex()}
        if kind in (list, tuple):
            return {"type": kind.__name__, "items": [self.node(item) for item in value]}
        if kind is dict:
            for key in value:
                if type(key) not in (str, int):
                    raise TypeError(f"save supports dict keys of type str or int, got {key!r}")
            return {"type": "dict", "keys": list(value), "values": [self.node(item) for item in value.values()]}
        if isinstance(value, (np.ndarray, np.generic)):
            return self.array(np.asarray(value))
        raise TypeError(f"save cannot save a {kind.__qualname__}: leaves must be arrays, None, bool, int, float or "
                        "str, and containers dict, list or tuple (save the fields of other classes instead)")

    def array(self, value: np.ndarray) -> dict:
        name = value.dtype.name
        if name not in _ARRAY_TYPES:
            raise TypeError(f"save supports float64, float32 and bool arrays, got {value.dtype}")
        blob = np.ascontiguousarray(value, dtype=_ARRAY_TYPES[name]).tobytes()
        node = {"type": "array", "dtype": name, "shape": [int(n) for n in value.shape], "offset": self.cursor,
                "nbytes": len(blob)}
        self.blobs.append(blob)
        self.cursor += len(blob)
        return node


def save(file, tree: Any) -> None:
    """Write `tree` to `file` (a path or a binary file object with `write`)."""
    writer = _Writer()
    header = json.dumps({"format": "quabla", "version": VERSION, "tree": writer.node(tree)}, allow_nan=False,
                        separators=(",", ":")).encode()
    parts = [MAGIC, _SIZE.pack(len(header)), header, *writer.blobs]
    if hasattr(file, "write"):
        _write_all(file, parts)
    else:
        with open(os.fspath(file), "wb") as handle:
            _write_all(handle, parts)


def _write_all(handle, parts) -> None:
    for part in parts:
        view = memoryview(part)
        while len(view):
            count = handle.write(view)
            if count is None or count <= 0 or count > len(view):
                raise OSError("save: the stream did not make valid write progress")
            view = view[count:]


def _bad(message: str) -> ValueError:
    return ValueError(f"malformed quabla save file header: {message}")


def _no_constants(token: str):
    raise _bad(f"{token} is not valid JSON")


def load(file) -> Any:
    """Read a tree written by `save` (or by the reference) from a path or a binary file object."""
    if hasattr(file, "read"):
        content = file.read()
    else:
        with open(os.fspath(file), "rb") as handle:
            content = handle.read()
    content = memoryview(content)
    start = len(MAGIC) + _SIZE.size
    if bytes(content[:len(MAGIC)]) != MAGIC:
        raise ValueError("not a quabla save file (bad magic bytes)")
    if len(content) < start:
        raise ValueError("truncated quabla save file (incomplete header size)")
    (size,) = _SIZE.unpack(content[len(MAGIC):start])
    if size > len(content) - start:
        raise ValueError("truncated quabla save file (incomplete header)")
    try:
        header = json.loads(bytes(content[start:start + size]), parse_constant=_no_constants)
    except (UnicodeDecodeError, json.JSONDecodeError, RecursionError) as error:
        raise _bad(str(error)) from None
    if not isinstance(header, dict) or header.get("format") != "quabla":
        raise _bad("not a quabla header")
    version = header.get("version")
    if type(version) is not int or version != VERSION:
        raise ValueError(f"unsupported quabla save file version {version!r}; this reader reads version {VERSION}")
    try:
        return _Reader(content[start + size:]).value(header.get("tree"))
    except RecursionError:
        raise _bad("tree nesting is too deep") from None


class _Reader:
    def __init__(self, data: memoryview) -> None:
        self.data = data

    def value(self, node: Any) -> Any:
        if not isinstance(node, dict):
            raise _bad(f"bad tree node {node!r}")
        kind = node.get("type")
        if kind == "none":
            return None
        if kind in ("bool", "int", "str"):
            value = node.get("value")
            if type(value).__name__ != kind:
                raise _bad(f"bad {kind} node {node!r}")
            return value
        if kind == "float":
            try:
                return float.fromhex(node["value"])
            except (KeyError, TypeError, ValueError, OverflowError):
                raise _bad(f"bad float node {node!r}") from None
        if kind in ("list", "tuple"):
            items = node.get("items")
            if type(items) is not list:
                raise _bad(f"bad {kind} node")
            decoded = [self.value(item) for item in items]
            return decoded if kind == "list" else tuple(decoded)
        if kind == "dict":
            keys, values = node.get("keys"), node.get("values")
            if (type(keys) is not list or type(values) is not list or len(keys) != len(values)
                    or any(type(key) not in (str, int) for key in keys) or len(set(keys)) != len(keys)):
                raise _bad("bad dict node")
            return {key: self.value(item) for key, item in zip(keys, values)}
        if kind == "array":
            return self.array(node)
        raise _bad(f"unknown node type {kind!r}")

    def array(self, node: dict) -> np.ndarray:
        name, shape, offset, nbytes = node.get("dtype"), node.get("shape"), node.get("offset"), node.get("nbytes")
        if (type(name) is not str or name not in _ARRAY_TYPES or type(shape) is not list
                or any(type(n) is not int or n < 0 for n in shape) or type(offset) is not int
                or type(nbytes) is not int or offset < 0):
            raise _bad(f"bad array node {node!r}")
        dtype = _ARRAY_TYPES[name]
        count = 1
        for n in shape:
            count *= n
        if nbytes != count * dtype.itemsize:
            raise _bad(f"{nbytes} bytes do not hold a {name} array of shape {shape}")
        if offset + nbytes > len(self.data):
            raise ValueError("truncated quabla save file (array data past the end of the file)")
        raw = self.data[offset:offset + nbytes]
        if name == "bool":
            octets = np.frombuffer(raw, dtype=np.uint8)
            if octets.size and int(octets.max()) > 1:
                raise ValueError("malformed quabla save file: bool data must contain only 0 or 1")
            return octets.astype(np.bool_).reshape(shape)
        # A copy in native byte order: aligned, writable, independent of the file buffer.
        return np.frombuffer(raw, dtype=dtype).astype(dtype.newbyteorder("="), copy=True).reshape(shape)
