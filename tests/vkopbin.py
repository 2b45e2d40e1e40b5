"""Writer of the reference's binary model format (.vkopbin), for the loader tests.

Layout as model/load.cpp:98-285 reads it: inputs, outputs, nodes (type, name, attribute dictionary with tags 0-4 of
model/load.hpp:241-275, inputs, outputs, dependencies, dependents), initializers, concurrent levels; every count and
length a little-endian u32."""
from __future__ import annotations

import struct


def _u32(v: int) -> bytes:
    return struct.pack("<I", v)


def _str(s: str) -> bytes:
    b = s.encode()
    return _u32(len(b)) + b


def _dims(d) -> bytes:
    return _u32(len(d)) + b"".join(_u32(int(x)) for x in d)


def _shapes(items) -> bytes:
    return _u32(len(items)) + b"".join(_str(n) + _dims(d) for n, d in items)


def _names(items) -> bytes:
    return _u32(len(items)) + b"".join(_str(n) for n in items)


def _attr(value) -> bytes:
    if isinstance(value, str):
        return b"\x00" + _str(value)
    if isinstance(value, bool) or isinstance(value, int):
        return b"\x01" + struct.pack("<q", int(value))
    if isinstance(value, float):
        return b"\x02" + struct.pack("<f", value)
    if isinstance(value, (list, tuple)) and all(isinstance(v, int) for v in value):
        return b"\x03" + _u32(len(value)) + b"".join(_u32(v) for v in value)
    if isinstance(value, (list, tuple)):
        return b"\x04" + _u32(len(value)) + b"".join(struct.pack("<f", float(v)) for v in value)
    raise TypeError(type(value))


def model_bytes(inputs, outputs, nodes, initializers=(), levels=None) -> bytes:
    """inputs / outputs: [(name, dims)]; nodes: [dict(op_type, name, attrs={}, inputs=[(name, dims)], outputs=[...],
    dependencies=[], dependents=[])]; initializers: [(name, dtype name, dims, raw bytes)]; levels: [[node names]]
    (default: one node per level, in order)."""
    out = _shapes(inputs) + _shapes(outputs) + _u32(len(nodes))
    for n in nodes:
        attrs = n.get("attrs", {})
        out += _str(n["op_type"]) + _str(n["name"]) + _u32(len(attrs))
        for k, v in attrs.items():
            out += _str(k) + _attr(v)
        out += _shapes(n["inputs"]) + _shapes(n["outputs"])
        out += _names(n.get("dependencies", [])) + _names(n.get("dependents", []))
    out += _u32(len(initializers))
    for name, dtype, dims, raw in initializers:
        out += _str(name) + _str(dtype) + _dims(dims) + struct.pack("<q", len(raw)) + raw
    if levels is None:
        levels = [[n["name"]] for n in nodes]
    out += _u32(len(levels))
    for level in levels:
        out += _names(level)
    return out


def write_model(path, *args, **kw) -> None:
    with open(path, "wb") as f:
        f.write(model_bytes(*args, **kw))
