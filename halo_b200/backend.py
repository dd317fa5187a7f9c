"""Host-side mirror of the reference's Backend interface for the matmul path, over the C ABI.

The names follow include/halo/backend/backend.h of the reference: a `CudaBackend` hands out
`Buffer`s and a `Stream`, operands are `TensorRef`s (buffer, byte offset, byte length, row stride),
`gemv(GemvArgs)` / `lm_head(LmHeadArgs)` / `get_rows(GetRowsArgs)` validate on the host and enqueue,
and failures raise `HaloError` carrying the reference's error class.  Everything else the interface
lists (norms, attention, ...) is not part of this backend and raises Unsupported; nothing ever falls
back to the CPU.  The C++ adapter in halo_b200/adapter implements the same mapping for C++ callers;
this module exists so that tests and the benchmark can drive the library from Python.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import capi
from .synth import F32, Q4_0, Q4_K, Q6_K, Q8_0, row_bytes  # noqa: F401

ARGMAX_RESULT_BYTES = 12  # kArgmaxResultBytes, backend.h:430


class HaloError(RuntimeError):
    """halo::Error: `code` is the class name of include/halo/core/error.h:15-26."""

    def __init__(self, status: int, message: str):
        self.status = status
        self.code = capi.ERROR_NAMES.get(status, "Backend")
        super().__init__(f"{self.code.upper()}_ERROR: {message}")


def _check(rc: int) -> None:
    if rc != 0:
        raise HaloError(rc, capi.last_error())


class Buffer:
    """Device memory owned by one backend (Buffer, backend.h:105-127). Never host-addressable."""

    def __init__(self, backend: "CudaBackend", ptr: int, nbytes: int, writable: bool):
        self._backend, self.ptr, self.nbytes, self.writable = backend, ptr, nbytes, writable

    def bytes(self) -> int:
        return self.nbytes

    def backend(self) -> "CudaBackend":
        return self._backend

    def free(self) -> None:
        if self.ptr:
            self._backend._free(self.ptr)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


@dataclass
class TensorRef:
    """Bytes [offset, offset + nbytes) of a buffer (nbytes 0 = to the end), row_stride 0 = dense (backend.h:129-155)."""
    buffer: Buffer | None = None
    offset: int = 0
    nbytes: int = 0
    row_stride: int = 0

    def empty(self) -> bool:
        return self.buffer is None

    @staticmethod
    def of(b: Buffer) -> "TensorRef":
        return TensorRef(b, 0, 0, 0)

    def view_bytes(self) -> int:
        if self.nbytes or self.buffer is None:
            return self.nbytes
        return max(self.buffer.nbytes - self.offset, 0)

    def shifted(self, delta: int) -> "TensorRef":
        if self.nbytes and delta >= self.nbytes:
            raise HaloError(capi.E_KERNEL, f"TensorRef::shifted: {delta} bytes past a {self.nbytes}-byte view")
        return TensorRef(self.buffer, self.offset + delta, 0 if self.nbytes == 0 else self.nbytes - delta, self.row_stride)

    def with_stride(self, stride: int) -> "TensorRef":
        return TensorRef(self.buffer, self.offset, self.nbytes, stride)


@dataclass
class GemvArgs:
    """GemvArgs (backend.h:283-314).  norm_w / norm_eps: the fused input norm, for one x row on the tensor-core skinny kernels and
    refused everywhere else; gates_*: the GDN gates epilogue, for F32 / Q8_0 weights on the fp32 kernels and refused everywhere else."""
    wtype: int = F32
    w: TensorRef = field(default_factory=TensorRef)
    x: TensorRef = field(default_factory=TensorRef)
    y: TensorRef = field(default_factory=TensorRef)
    rows: int = 0
    cols: int = 0
    n_vec: int = 1
    variant_id: int = 0
    norm_w: TensorRef = field(default_factory=TensorRef)
    norm_eps: float = 1e-6
    allow_gemm: bool = False
    gates_n_v: int = 0
    gates_dt_bias: TensorRef = field(default_factory=TensorRef)
    gates_a: TensorRef = field(default_factory=TensorRef)
    #: cuda extension: the call may not touch context scratch (the statically partitioned kernels; what
    #: halo_cuda_lm_head_noalloc computes)
    no_scratch: bool = False


@dataclass
class LmHeadArgs:
    """LmHeadArgs (backend.h:437-460); row_offset is the vocabulary offset of a column-split shard."""
    gemv: GemvArgs = field(default_factory=GemvArgs)
    result: TensorRef = field(default_factory=TensorRef)
    valid_rows: int = 0
    ids: TensorRef = field(default_factory=TensorRef)
    row_offset: int = 0


@dataclass
class GetRowsArgs:
    """GetRowsArgs (backend.h:251-262); ids may be empty (rows 0..n_ids-1)."""
    type: int = F32
    table: TensorRef = field(default_factory=TensorRef)
    ids: TensorRef = field(default_factory=TensorRef)
    out: TensorRef = field(default_factory=TensorRef)
    n_rows: int = 0
    cols: int = 0
    n_ids: int = 0


class Stream:
    """Ordered work queue (Stream, backend.h:494-506)."""

    def __init__(self, backend: "CudaBackend", handle: int | None = None):
        self._backend = backend
        self._own = handle is None
        if handle is None:
            h = C.c_void_p()
            _check(backend.lib.halo_cuda_stream_create(backend.ctx, C.byref(h)))
            handle = h.value or 0
        self.handle = handle

    def submit(self) -> None:
        pass

    def wait(self, timeout_ns: int = 0) -> None:
        _check(self._backend.lib.halo_cuda_stream_sync(self._backend.ctx, self.handle, timeout_ns))

    def abort(self) -> None:
        try:
            self.wait()
        except HaloError:
            pass

    def __del__(self):
        try:
            if self._own and self.handle:
                self._backend.lib.halo_cuda_stream_destroy(self._backend.ctx, self.handle)
        except Exception:
            pass


class CudaBackend:
    """The `cuda` backend: MATMUL, LM_HEAD, GET_ROWS, COPY, upload / download."""

    def __init__(self, device: int = 0):
        self.lib = capi.load()
        ctx = C.c_void_p()
        _check(self.lib.halo_cuda_ctx_create(device, C.byref(ctx)))
        self.ctx = ctx
        self.device = device

    def close(self) -> None:
        if getattr(self, "ctx", None):
            self.lib.halo_cuda_ctx_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- identity -------------------------------------------------------------------------------
    def kind(self) -> str:
        return "cuda"

    def info(self) -> capi.DeviceInfo:
        info = capi.DeviceInfo()
        _check(self.lib.halo_cuda_device_info(self.ctx, C.byref(info)))
        return info

    def describe(self) -> str:
        i = self.info()
        return f"cuda {i.name.decode()} ({i.arch.decode()}, {i.sm_count} SMs)"

    def lost(self) -> bool:
        return bool(self.lib.halo_cuda_ctx_lost(self.ctx))

    def scratch_bytes(self) -> int:
        """Context scratch the kernels have allocated on demand so far."""
        n = C.c_uint64()
        _check(self.lib.halo_cuda_ctx_scratch_bytes(self.ctx, C.byref(n)))
        return n.value

    def variants(self, op: int) -> list[tuple[int, str, int]]:
        n = C.c_uint32()
        arr = (capi.Variant * 16)()
        _check(self.lib.halo_cuda_variants(op, arr, 16, C.byref(n)))
        return [(arr[i].id, arr[i].name.decode(), arr[i].family) for i in range(n.value)]

    # ---- memory ----------------------------------------------------------------------------------
    def allocate(self, nbytes: int, zero: bool = True, shareable: bool = False) -> Buffer:
        """Zero-filled device memory from the context's pool (Backend::allocate, backend.h:523); `shareable` takes it from the
        driver instead, which exporting it to another process needs."""
        p = C.c_void_p()
        _check(self.lib.halo_cuda_malloc(self.ctx, nbytes, (1 if zero else 0) | (2 if shareable else 0), C.byref(p)))
        return Buffer(self, p.value or 0, nbytes, True)

    def _free(self, ptr: int) -> None:
        if getattr(self, "ctx", None):
            self.lib.halo_cuda_free(self.ctx, ptr)

    def import_host(self, array):
        raise HaloError(capi.E_UNSUPPORTED, "import_host: a device backend cannot alias caller memory; allocate + upload instead")

    def import_host_readonly(self, array: np.ndarray, stream: Stream | None = None) -> Buffer:
        """Copies the bytes to the device (weights are copied at import, as on the reference's device backends)."""
        a = np.ascontiguousarray(array)
        buf = self.allocate(a.nbytes, zero=False)
        buf.writable = False
        s = stream or self._default_stream()
        _check(self.lib.halo_cuda_memcpy_h2d_async(self.ctx, buf.ptr, a.ctypes.data, a.nbytes, s.handle))
        s.wait()
        return buf

    def create_stream(self) -> Stream:
        return Stream(self)

    def wrap_stream(self, cuda_stream: int) -> Stream:
        """A Stream over an existing cudaStream_t (e.g. torch's current stream), not owned."""
        return Stream(self, cuda_stream)

    def _default_stream(self) -> Stream:
        if not hasattr(self, "_stream0"):
            self._stream0 = Stream(self)
        return self._stream0

    def _resolve(self, ref: TensorRef, need: int, name: str, op: str, write: bool = False) -> int:
        if ref.empty():
            return 0
        b = ref.buffer
        if b.backend() is not self:
            raise HaloError(capi.E_KERNEL, f"{op}: operand {name} belongs to another backend")
        if write and not b.writable:
            raise HaloError(capi.E_KERNEL, f"{op}: output {name} is read-only")
        if ref.offset > b.nbytes:
            raise HaloError(capi.E_KERNEL, f"{op}: operand {name} offset {ref.offset} past buffer end {b.nbytes}")
        avail = b.nbytes - ref.offset
        limit = ref.nbytes if ref.nbytes else avail
        if limit > avail:
            raise HaloError(capi.E_KERNEL, f"{op}: operand {name} range exceeds buffer of {b.nbytes} bytes")
        if need > limit:
            raise HaloError(capi.E_KERNEL, f"{op}: operand {name} needs {need} bytes, view has {limit}")
        return b.ptr + ref.offset

    @staticmethod
    def _extent(n: int, row: int, stride: int) -> int:
        return 0 if n == 0 else (n - 1) * (stride or row) + row

    def upload(self, s: Stream, dst: TensorRef, src: np.ndarray) -> None:
        a = np.ascontiguousarray(src)
        p = self._resolve(dst, a.nbytes, "dst", "upload", write=True)
        s._keep = getattr(s, "_keep", []) + [a]  # src must stay valid until wait()
        _check(self.lib.halo_cuda_memcpy_h2d_async(self.ctx, p, a.ctypes.data, a.nbytes, s.handle))

    def download(self, s: Stream, src: TensorRef, dst: np.ndarray) -> None:
        assert dst.flags.c_contiguous
        p = self._resolve(src, dst.nbytes, "src", "download")
        _check(self.lib.halo_cuda_memcpy_d2h_async(self.ctx, dst.ctypes.data, p, dst.nbytes, s.handle))

    def copy(self, s: Stream, src: TensorRef, dst: TensorRef, nbytes: int) -> None:
        ps = self._resolve(src, nbytes, "src", "COPY")
        pd = self._resolve(dst, nbytes, "dst", "COPY", write=True)
        _check(self.lib.halo_cuda_memcpy_d2d_async(self.ctx, pd, ps, nbytes, s.handle))

    # ---- ops ---------------------------------------------------------------------------------------
    def _gemv_struct(self, a: GemvArgs, op: str, y_optional: bool) -> capi.Gemv:
        if not a.norm_w.empty() and op != "MATMUL":
            raise HaloError(capi.E_UNSUPPORTED, f"{op}: a fused norm (GemvArgs::norm_w) is for MATMUL only")
        if a.gates_n_v != 0 and (op != "MATMUL" or not a.norm_w.empty()):
            raise HaloError(capi.E_UNSUPPORTED, f"{op}: the GDN gates epilogue (GemvArgs::gates) is for MATMUL without a fused norm")
        rb = C.c_uint64()
        if a.variant_id in capi.REPACKED_VARIANTS:  # W is in the repacked row layout
            _check(self.lib.halo_cuda_repacked_row_bytes(a.wtype, a.cols, C.byref(rb)))
        else:
            _check(self.lib.halo_cuda_row_bytes(a.wtype, a.cols, C.byref(rb)))
        g = capi.Gemv()
        g.wtype, g.variant_id = a.wtype, a.variant_id
        g.w = self._resolve(a.w, self._extent(a.rows, rb.value, a.w.row_stride), "w", op) or None
        g.w_stride = a.w.row_stride
        g.x = self._resolve(a.x, self._extent(a.n_vec, a.cols * 4, a.x.row_stride), "x", op) or None
        g.x_stride = a.x.row_stride
        g.y = self._resolve(a.y, self._extent(a.n_vec, a.rows * 4, a.y.row_stride), "y", op, write=True) or None
        g.y_stride = a.y.row_stride
        g.rows, g.cols, g.n_vec = a.rows, a.cols, a.n_vec
        g.flags = (capi.FLAG_ALLOW_GEMM if a.allow_gemm else 0) | (capi.FLAG_NO_SCRATCH if a.no_scratch else 0)
        return g

    def gemv(self, s: Stream, a: GemvArgs) -> None:
        g = self._gemv_struct(a, "MATMUL", False)
        if a.gates_n_v != 0:
            db = self._resolve(a.gates_dt_bias, a.gates_n_v * 4, "gates.dt_bias", "MATMUL")
            ga = self._resolve(a.gates_a, a.gates_n_v * 4, "gates.a", "MATMUL")
            _check(self.lib.halo_cuda_gemv_gated(self.ctx, C.byref(g), db, ga, a.gates_n_v, s.handle))
            return
        if not a.norm_w.empty():
            nw = self._resolve(a.norm_w, a.cols * 4, "norm_w", "MATMUL")
            _check(self.lib.halo_cuda_gemv_normed(self.ctx, C.byref(g), nw, a.norm_eps, s.handle))
            return
        _check(self.lib.halo_cuda_gemv(self.ctx, C.byref(g), s.handle))

    def resolve_variant(self, a: GemvArgs) -> int:
        g = self._gemv_struct(a, "MATMUL", False)
        v = C.c_uint32()
        _check(self.lib.halo_cuda_gemv_resolve(self.ctx, C.byref(g), C.byref(v)))
        return v.value

    def lm_head(self, s: Stream, a: LmHeadArgs) -> None:
        h = capi.LmHead()
        h.gemv = self._gemv_struct(a.gemv, "LM_HEAD", True)
        h.result = self._resolve(a.result, a.gemv.n_vec * ARGMAX_RESULT_BYTES, "result", "LM_HEAD", write=True) or None
        h.ids = self._resolve(a.ids, a.gemv.n_vec * 4, "ids", "LM_HEAD", write=True) or None
        h.valid_rows, h.row_offset = a.valid_rows, a.row_offset
        _check(self.lib.halo_cuda_lm_head(self.ctx, C.byref(h), s.handle))

    def lm_head_noalloc(self, s: Stream, a: LmHeadArgs) -> None:
        """lm_head for hosts that may not allocate device memory mid-run: same operands, logits buffer required,
        argmax partials in the library's fixed 64 KiB scratch (halo_cuda_lm_head_noalloc)."""
        h = capi.LmHead()
        h.gemv = self._gemv_struct(a.gemv, "LM_HEAD", False)
        h.result = self._resolve(a.result, a.gemv.n_vec * ARGMAX_RESULT_BYTES, "result", "LM_HEAD", write=True) or None
        h.ids = self._resolve(a.ids, a.gemv.n_vec * 4, "ids", "LM_HEAD", write=True) or None
        h.valid_rows, h.row_offset = a.valid_rows, a.row_offset
        _check(self.lib.halo_cuda_lm_head_noalloc(self.ctx, C.byref(h), s.handle))

    def get_rows(self, s: Stream, a: GetRowsArgs, status: Buffer | None = None) -> None:
        rb = C.c_uint64()
        _check(self.lib.halo_cuda_row_bytes(a.type, a.cols, C.byref(rb)))
        g = capi.GetRows()
        g.type = a.type
        g.table = self._resolve(a.table, self._extent(a.n_rows, rb.value, a.table.row_stride), "table", "GET_ROWS") or None
        g.table_stride = a.table.row_stride
        g.ids = self._resolve(a.ids, a.n_ids * 4, "ids", "GET_ROWS") or None
        g.out = self._resolve(a.out, self._extent(a.n_ids, a.cols * 4, a.out.row_stride), "out", "GET_ROWS", write=True) or None
        g.out_stride = a.out.row_stride
        g.n_rows, g.cols, g.n_ids = a.n_rows, a.cols, a.n_ids
        g.status = status.ptr if status is not None else None
        _check(self.lib.halo_cuda_get_rows(self.ctx, C.byref(g), s.handle))

    def repacked_row_bytes(self, wtype: int, cols: int) -> int:
        rb = C.c_uint64()
        _check(self.lib.halo_cuda_repacked_row_bytes(wtype, cols, C.byref(rb)))
        return rb.value

    def repacked_variant(self, wtype: int, cols: int) -> int:
        """The variant id a repacked tensor of this type and (largest local) K travels with."""
        v = C.c_uint32()
        _check(self.lib.halo_cuda_repacked_variant(wtype, cols, C.byref(v)))
        return v.value

    def repack(self, s: Stream, wtype: int, src: TensorRef, rows: int, cols: int) -> Buffer:
        """Raw GGUF rows -> a new read-only buffer in the repacked layout gemv_mma_r reads (what a loader does once per
        weight, like tensor::gemv_repack for the reference's Vulkan backend)."""
        raw = C.c_uint64()
        _check(self.lib.halo_cuda_row_bytes(wtype, cols, C.byref(raw)))
        prb = self.repacked_row_bytes(wtype, cols)
        p = self._resolve(src, self._extent(rows, raw.value, src.row_stride), "src", "repack")
        dst = self.allocate(max(rows * prb, 16), zero=False)
        _check(self.lib.halo_cuda_repack_rows(self.ctx, wtype, p, src.row_stride, dst.ptr, 0, rows, cols, s.handle))
        dst.writable = False
        return dst

    def plan_set(self, wtype: int, rows: int, cols: int, n_vec_lo: int, n_vec_hi: int, variant_id: int) -> None:
        _check(self.lib.halo_cuda_plan_set(self.ctx, wtype, rows, cols, n_vec_lo, n_vec_hi, variant_id))

    def plan_clear(self) -> None:
        _check(self.lib.halo_cuda_plan_clear(self.ctx))

    def _unsupported(self, *_a, **_k):
        raise HaloError(capi.E_UNSUPPORTED, "this op is not part of the cuda matmul backend")

    rms_norm = add_rms_norm = gdn_gates = conv1d_silu = gated_delta_rule = gated_rms_norm = _unsupported
    partial_rope = kv_write = attention = swiglu = mul_sigmoid = add = argmax = top_k = _unsupported


def decode_argmax(words: np.ndarray) -> list[tuple[int, float]]:
    """decode_argmax (src/backend/backend.cpp:83-99): a poisoned vector decodes to (-1, NaN)."""
    w = np.ascontiguousarray(words, np.uint32).reshape(-1, 3)
    out = []
    for idx, bits, nan in w:
        if nan != 0:
            out.append((-1, float("nan")))
        else:
            out.append((int(idx) - (1 << 32) if int(idx) >= (1 << 31) else int(idx), float(np.array([bits], np.uint32).view(np.float32)[0])))
    return out
