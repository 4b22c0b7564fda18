"""A minimal GGUF v2/v3 writer for the tests (the byte layout the reference's parser tests
build by hand, src/parser.rs:190-207, extended with a data section)."""
import struct

import numpy as np

TYPE_IDS = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "array": 9, "u64": 10,
            "i64": 11, "f64": 12}
_FMT = {"u8": "<B", "i8": "<b", "u16": "<H", "i16": "<h", "u32": "<I", "i32": "<i", "f32": "<f", "bool": "<B", "u64": "<Q",
        "i64": "<q", "f64": "<d"}


def gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def value(kind: str, v) -> bytes:
    if kind == "str":
        return gstr(v)
    if kind == "array":
        elem_kind, items = v
        return struct.pack("<IQ", TYPE_IDS[elem_kind], len(items)) + b"".join(value(elem_kind, i) for i in items)
    return struct.pack(_FMT[kind], v)


def header(version: int, tensor_count: int, kv_count: int) -> bytes:
    return b"GGUF" + struct.pack("<IQQ", version, tensor_count, kv_count)


def build(version, metadata, tensors):
    """metadata: list of (key, kind, value); tensors: list of (name, ggml_type, dims, raw bytes).
    Returns the file bytes; tensor data is laid out at 32-byte aligned offsets."""
    tensors = [(n, t, d, raw if isinstance(raw, (bytes, bytearray)) else np.ascontiguousarray(raw).tobytes())
               for n, t, d, raw in tensors]
    out = bytearray(header(version, len(tensors), len(metadata)))
    for key, kind, v in metadata:
        out += gstr(key) + struct.pack("<I", TYPE_IDS[kind]) + value(kind, v)
    offsets, off = [], 0
    for name, ggml_type, dims, raw in tensors:
        offsets.append(off)
        off = (off + len(raw) + 31) & ~31
    for (name, ggml_type, dims, raw), o in zip(tensors, offsets):
        out += gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", ggml_type, o)
    out += b"\0" * ((-len(out)) % 32)
    for (name, ggml_type, dims, raw), o in zip(tensors, offsets):
        assert len(out) % 32 == 0
        out += raw
        out += b"\0" * ((-len(out)) % 32)
    return bytes(out)
