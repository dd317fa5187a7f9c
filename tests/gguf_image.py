"""A minimal GGUF v3 image builder for the loader tests: well-formed files and deliberately damaged ones.

It follows the published container layout (little-endian): magic, version, tensor count, metadata count, metadata
pairs, tensor infos, padding to the alignment, tensor data.  Every piece can be overridden, so a test can state
exactly which field it breaks.  The reference tests its parser the same way, with an in-memory writer
(tests/unit/model/gguf_builder.h:22-279).
"""
from __future__ import annotations

import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def string(s: bytes | str) -> bytes:
    b = s.encode() if isinstance(s, str) else s
    return struct.pack("<Q", len(b)) + b


def value(vtype: int, v) -> bytes:
    if vtype in _FMT:
        return struct.pack(_FMT[vtype], v)
    if vtype == STRING:
        return string(v)
    if vtype == ARRAY:
        elem, items = v
        return struct.pack("<IQ", elem, len(items)) + b"".join(value(elem, i) for i in items)
    raise ValueError(vtype)


def kv(key: str, vtype: int, v) -> bytes:
    return string(key) + struct.pack("<I", vtype) + value(vtype, v)


def tensor_info(name: str | bytes, ne: list[int], type_id: int, offset: int) -> bytes:
    return string(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", e) for e in ne) + struct.pack("<IQ", type_id, offset)


def image(kvs: list[bytes], infos: list[bytes], data: bytes = b"", alignment: int = 32, version: int = 3, magic: bytes = b"GGUF",
          n_tensors: int | None = None, n_kv: int | None = None) -> bytes:
    head = magic + struct.pack("<IQQ", version, len(infos) if n_tensors is None else n_tensors, len(kvs) if n_kv is None else n_kv)
    head += b"".join(kvs) + b"".join(infos)
    pad = (-len(head)) % alignment
    return head + b"\0" * pad + data


def place(tensors: list[tuple[str, list[int], int, bytes]], alignment: int = 32) -> tuple[list[bytes], bytes]:
    """(name, ne, type, bytes) -> tensor infos with aligned offsets, and the data section."""
    infos, data = [], b""
    for name, ne, type_id, raw in tensors:
        data += b"\0" * ((-len(data)) % alignment)
        infos.append(tensor_info(name, ne, type_id, len(data)))
        data += bytes(raw)
    return infos, data


def random_bytes(seed: int, n: int) -> bytes:
    return np.random.default_rng(seed).integers(0, 256, n, dtype=np.uint8).tobytes()
