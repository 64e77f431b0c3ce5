"""Builds GGUF files in memory for the container tests (the reference has no writer; the layout is the one
`GgufFile::parse` reads: src/gguf.rs:411-482)."""
import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _value(vtype: int, v) -> bytes:
    if vtype == STR:
        return _string(v)
    if vtype == ARR:
        elem_type, items = v
        return struct.pack("<IQ", elem_type, len(items)) + b"".join(_value(elem_type, x) for x in items)
    return struct.pack(_FMT[vtype], v)


def build(kvs, tensors, version=3, alignment=None, magic=0x46554747) -> bytes:
    """kvs: [(key, vtype, value)]; tensors: [(name, file_shape, ggml_type, raw_bytes)].  Returns the file."""
    kvs = list(kvs)
    if alignment is not None:
        kvs.append(("general.alignment", U32, alignment))
    align = alignment or 32
    head = struct.pack("<IIQQ", magic, version, len(tensors), len(kvs))
    for key, vtype, v in kvs:
        head += _string(key) + struct.pack("<I", vtype) + _value(vtype, v)
    offsets, blob = [], b""
    for _, _, _, raw in tensors:
        pad = (-len(blob)) % align
        blob += b"\0" * pad
        offsets.append(len(blob))
        blob += bytes(raw)
    for (name, shape, dtype, _), off in zip(tensors, offsets):
        head += _string(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        head += struct.pack("<IQ", dtype, off)
    head += b"\0" * ((-len(head)) % align)
    return head + blob
