"""Writes small GGUF v3 files for the tests, the way the reference's own test does
(.github/runtime/suite.rs:127-214: header, metadata pairs, tensor descriptors, data section padded to 32)."""
from __future__ import annotations

import struct

import numpy as np

KIND_U8, KIND_I8, KIND_U16, KIND_I16, KIND_U32, KIND_I32, KIND_F32, KIND_BOOL, KIND_STRING, KIND_ARRAY, KIND_U64, KIND_I64, KIND_F64 = range(13)


def _text(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(kind: int, v) -> bytes:
    fmt = {KIND_U8: "<B", KIND_I8: "<b", KIND_U16: "<H", KIND_I16: "<h", KIND_U32: "<I", KIND_I32: "<i", KIND_F32: "<f", KIND_U64: "<Q", KIND_I64: "<q",
           KIND_F64: "<d"}
    if kind in fmt:
        return struct.pack(fmt[kind], v)
    if kind == KIND_BOOL:
        return bytes([1 if v else 0])
    if kind == KIND_STRING:
        return _text(v)
    if kind == KIND_ARRAY:
        item_kind, items = v
        return struct.pack("<IQ", item_kind, len(items)) + b"".join(_value(item_kind, i) for i in items)
    raise ValueError(kind)


def write_gguf(path, metadata, tensors, alignment: int = 32, version: int = 3, declare_alignment: bool = False) -> None:
    """metadata: [(key, kind, value)]; tensors: [(name, shape (k first, as GGUF stores it), ggml_type, bytes)]."""
    md = list(metadata)
    if declare_alignment:
        md.append(("general.alignment", KIND_U32, alignment))
    out = bytearray(b"GGUF") + struct.pack("<IQQ", version, len(tensors), len(md))
    for key, kind, value in md:
        out += _text(key) + struct.pack("<I", kind) + _value(kind, value)
    data = bytearray()
    for name, shape, ggml_type, payload in tensors:
        out += _text(name) + struct.pack("<I", len(shape))
        for extent in shape:
            out += struct.pack("<Q", extent)
        out += struct.pack("<IQ", ggml_type, len(data))
        data += bytes(np.ascontiguousarray(payload).view(np.uint8).reshape(-1))
        while len(data) % alignment:
            data.append(0)
    while len(out) % alignment:
        out.append(0)
    with open(path, "wb") as f:
        f.write(bytes(out) + bytes(data))
