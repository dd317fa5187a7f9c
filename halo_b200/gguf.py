"""GGUF container index and the file -> device upload of matmul operands, over the C ABI of include/halo_cuda_gguf.h.

The Python face of what the reference does in model::GgufFile (include/halo/model/gguf.h:133-199) and in
Impl::make_mat / try_repack (src/models/qwen35.cpp:301-346).  Parsing and the staged upload are native; this module
only mirrors their interface.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from . import backend as hb
from . import capi


def _check(rc: int) -> None:
    if rc != 0:
        raise hb.HaloError(rc, capi.last_error())


@dataclass(frozen=True)
class TensorInfo:
    """GgufTensorInfo (gguf.h:83-100): ne in ggml order, ne[0] contiguous; a projection is ne = (cols, rows)."""
    index: int
    name: str
    n_dims: int
    type: int
    ne: tuple[int, int, int, int]
    offset: int
    n_elements: int
    n_bytes: int
    supported: bool

    def rows(self) -> int:
        return self.ne[1] * self.ne[2] * self.ne[3]


class GgufFile:
    """An immutable parsed container.  `open` maps the file; `parse` reads an image the object keeps alive."""

    def __init__(self, handle: int, keep=None):
        self._h, self._keep, self.lib = handle, keep, capi.load()
        info = capi.GgufInfo()
        _check(self.lib.halo_gguf_info(self._h, C.byref(info)))
        self.version, self.alignment = info.version, info.alignment
        self.n_kv, self.n_tensors = info.n_kv, info.n_tensors
        self.header_size, self.data_offset, self.file_size = info.header_size, info.data_offset, info.file_size

    @staticmethod
    def open(path: str | Path) -> "GgufFile":
        h = C.c_void_p()
        _check(capi.load().halo_gguf_open(str(path).encode(), C.byref(h)))
        return GgufFile(h.value)

    @staticmethod
    def parse(image: bytes | bytearray | np.ndarray) -> "GgufFile":
        arr = np.frombuffer(image, np.uint8) if not isinstance(image, np.ndarray) else np.ascontiguousarray(image).view(np.uint8).reshape(-1)
        h = C.c_void_p()
        _check(capi.load().halo_gguf_parse(C.c_void_p(arr.ctypes.data if arr.size else 0), arr.size, C.byref(h)))
        return GgufFile(h.value, keep=arr)

    def close(self) -> None:
        if self._h:
            self.lib.halo_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- metadata: None when the key is absent, HaloError(Model) when its type cannot represent the request ----
    def _get(self, fn, ctype, key: str):
        v, found = ctype(), C.c_int()
        _check(fn(self._h, key.encode(), C.byref(v), C.byref(found)))
        return v.value if found.value else None

    def get_uint(self, key: str) -> int | None:
        return self._get(self.lib.halo_gguf_kv_u64, C.c_uint64, key)

    def get_int(self, key: str) -> int | None:
        return self._get(self.lib.halo_gguf_kv_i64, C.c_int64, key)

    def get_float(self, key: str) -> float | None:
        return self._get(self.lib.halo_gguf_kv_f64, C.c_double, key)

    def get_string(self, key: str) -> str | None:
        n, found = C.c_uint64(), C.c_int()
        _check(self.lib.halo_gguf_kv_string(self._h, key.encode(), None, 0, C.byref(n), C.byref(found)))
        if not found.value:
            return None
        buf = C.create_string_buffer(n.value + 1)
        _check(self.lib.halo_gguf_kv_string(self._h, key.encode(), buf, n.value + 1, C.byref(n), C.byref(found)))
        return buf.raw[:n.value].decode(errors="replace")

    # ---- tensors ----
    def tensor(self, index: int) -> TensorInfo:
        t = capi.GgufTensor()
        _check(self.lib.halo_gguf_tensor(self._h, index, C.byref(t)))
        return TensorInfo(index, t.name.decode(errors="replace"), t.n_dims, t.type, tuple(t.ne), t.offset, t.n_elements, t.n_bytes,
                          bool(t.supported))

    def tensors(self) -> list[TensorInfo]:
        return [self.tensor(i) for i in range(self.n_tensors)]

    def find_tensor(self, name: str) -> TensorInfo | None:
        idx, found = C.c_uint64(), C.c_int()
        _check(self.lib.halo_gguf_find(self._h, name.encode(), C.byref(idx), C.byref(found)))
        return self.tensor(idx.value) if found.value else None

    def tensor_data(self, t: TensorInfo) -> np.ndarray:
        """The tensor's bytes as a read-only view into the mapping (valid while this object lives)."""
        p, n = C.c_void_p(), C.c_uint64()
        _check(self.lib.halo_gguf_tensor_data(self._h, t.index, C.byref(p), C.byref(n)))
        if n.value == 0:
            return np.empty(0, np.uint8)
        a = np.ctypeslib.as_array((C.c_uint8 * n.value).from_address(p.value))
        a.flags.writeable = False
        return a


@dataclass
class DeviceMatrix:
    """A device-resident matmul operand (the reference's Mat, src/models/qwen35.cpp:52-67): what GemvArgs takes."""
    buf: hb.Buffer | None
    wtype: int
    variant_id: int
    rows: int
    cols: int
    row_stride: int
    row0: int
    k0: int

    def ref(self) -> hb.TensorRef:
        return hb.TensorRef(self.buf, 0, 0, self.row_stride)


def _how(split: int, rank: int, world: int, repack: bool, staging_bytes: int) -> capi.Upload:
    u = capi.Upload()
    u.split, u.rank, u.world, u.repack, u.staging_bytes = split, rank, world, int(repack), staging_bytes
    return u


def matrix_share(wtype: int, rows: int, cols: int, split: int = capi.SPLIT_NONE, rank: int = 0, world: int = 1,
                 repack: bool = False) -> DeviceMatrix:
    """The extents of one rank's share, computed without a device."""
    m = capi.Matrix()
    _check(capi.load().halo_cuda_matrix_share(wtype, rows, cols, C.byref(_how(split, rank, world, repack, 0)), C.byref(m)))
    return DeviceMatrix(None, m.wtype, m.variant_id, m.rows, m.cols, m.w_stride, m.row0, m.k0)


def upload_matrix(be: hb.CudaBackend, s: hb.Stream, f: GgufFile, t: TensorInfo, split: int = capi.SPLIT_NONE, rank: int = 0,
                  world: int = 1, repack: bool = False, staging_bytes: int = 0) -> DeviceMatrix:
    """Tensor `t` of `f`, or this rank's share of it, as a read-only device buffer; ready in the order of stream `s`."""
    m = capi.Matrix()
    _check(be.lib.halo_cuda_upload_matrix(be.ctx, f._h, t.index, C.byref(_how(split, rank, world, repack, staging_bytes)), s.handle,
                                          C.byref(m)))
    buf = hb.Buffer(be, m.w, m.bytes, writable=False) if m.w else None
    return DeviceMatrix(buf, m.wtype, m.variant_id, m.rows, m.cols, m.w_stride, m.row0, m.k0)


def write_gguf(path: str | Path, tensors: list[tuple[str, int, int, int, np.ndarray]], metadata: dict[str, int | float | str] | None = None,
               alignment: int = 32) -> None:
    """Writes a GGUF v3 container of 2-D tensors (name, ggml type, rows, cols, raw row bytes) and scalar / string metadata:
    enough to produce synthetic model files for the loader (the published layout; integers as UINT32, floats as FLOAT32)."""
    import struct

    def s(b: str) -> bytes:
        e = b.encode()
        return struct.pack("<Q", len(e)) + e

    meta = dict(metadata or {})
    if alignment != 32:
        meta["general.alignment"] = alignment
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, v in meta.items():
        if isinstance(v, str):
            head += s(k) + struct.pack("<I", 8) + s(v)
        elif isinstance(v, float):
            head += s(k) + struct.pack("<If", 6, v)
        else:
            head += s(k) + struct.pack("<II", 4, v)
    offset, offsets = 0, []
    for name, t, rows, cols, raw in tensors:
        offset = (offset + alignment - 1) // alignment * alignment
        offsets.append(offset)
        head += s(name) + struct.pack("<IQQIQ", 2, cols, rows, t, offset)
        offset += int(np.asarray(raw).nbytes)
    with open(path, "wb") as out:
        out.write(head)
        out.write(b"\0" * ((-len(head)) % alignment))
        pos = 0
        for (name, t, rows, cols, raw), off in zip(tensors, offsets):
            out.write(b"\0" * (off - pos))
            a = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
            out.write(a.data)
            pos = off + a.size


def host_share(f: GgufFile, t: TensorInfo, split: int = capi.SPLIT_NONE, rank: int = 0, world: int = 1) -> tuple[DeviceMatrix, np.ndarray]:
    """One rank's share of matrix `t` as host bytes [rows, local row bytes] (a view into the mapping for whole rows, a copy for a
    K range), with its extents: what halo_cuda_upload_matrix would bring to the device.  For tools and the CPU tests."""
    m = matrix_share(t.type, t.ne[1], t.ne[0], split, rank, world)
    src_row = t.n_bytes // t.ne[1] if t.ne[1] else 0
    data = f.tensor_data(t).reshape(t.ne[1], src_row) if t.ne[1] else np.empty((0, 0), np.uint8)
    if m.rows == 0 or m.cols == 0:
        return m, np.empty((m.rows, 0), np.uint8)
    local = m.row_stride
    byte0 = (m.k0 * src_row) // t.ne[0]
    return m, data[m.row0:m.row0 + m.rows, byte0:byte0 + local]
