"""Writes GGUF (version 3) files for the tests: metadata scalars, strings and arrays, a tensor table, aligned tensor data.
Test infrastructure; the layout is llama.cpp's published one (magic, version, counts, key-value pairs, tensor infos, data)."""
import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
GGML = dict(F32=0, F16=1, Q8_0=8, Q4_K=12, Q5_K=13, Q6_K=14, BF16=30)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _string(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(kind, value):
    if kind == STRING:
        return _string(value)
    if kind == ARRAY:
        inner, items = value
        return struct.pack("<IQ", inner, len(items)) + b"".join(_value(inner, v) for v in items)
    return struct.pack(_SCALAR[kind], value)


def write(path, metadata, tensors, alignment=32, version=3, magic=b"GGUF"):
    """metadata: list of (key, kind, value); tensors: list of (name, ggml type id, dims fastest first, bytes-like data)."""
    head = magic + struct.pack("<IQQ", version, len(tensors), len(metadata))
    for key, kind, value in metadata:
        head += _string(key) + struct.pack("<I", kind) + _value(kind, value)
    offset, infos, blobs = 0, b"", []
    for name, kind, dims, data in tensors:
        data = bytes(np.ascontiguousarray(data).view(np.uint8).reshape(-1)) if not isinstance(data, (bytes, bytearray)) else bytes(data)
        infos += _string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", kind, offset)
        blobs.append((offset, data))
        offset = (offset + len(data) + alignment - 1) // alignment * alignment
    head += infos
    start = (len(head) + alignment - 1) // alignment * alignment
    out = bytearray(head) + bytearray(start - len(head))
    for off, data in blobs:
        out += bytearray(start + off - len(out)) + data
    with open(path, "wb") as f:
        f.write(out)
    return start
