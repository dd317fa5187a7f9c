"""CPU oracle for the quantized weight matmul path.  TEST INFRASTRUCTURE ONLY.

Two checkers live here, both reached through ctypes:

* ``Oracle``    -- ``liboracle.so``, the plain-C restatement in ``halo_oracle.c`` (kind "port").
* ``Reference`` -- ``_ref/libhalo_ref.so``, the unmodified reference CPU backend compiled from
  the reference tree's own sources (kind "reference"); present only where it was built.

Only the test-suite, the smoke check and the CPU-baseline / reference legs of the benchmark may
import this package.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "liboracle.so"
REF_SO = HERE / "_ref" / "libhalo_ref.so"

F32, Q4_0, Q8_0, Q4_K, Q6_K = 0, 2, 8, 12, 14

_u8p = C.POINTER(C.c_uint8)


def find_ref_root() -> Path | None:
    """The reference source tree: $HALO_REF_ROOT, else a directory `reference` next to this repository; None when neither holds one."""
    env = os.environ.get("HALO_REF_ROOT")
    for root in ([Path(env)] if env else []) + [HERE.parent.parent / "reference"]:
        if (root / "src" / "backend" / "cpu_backend.cpp").exists():
            return root
    return None


def build(ref_root: str | None = None) -> None:
    """Compile the C restatement, and the reference library when the reference tree exists."""
    subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    root = Path(ref_root) if ref_root else find_ref_root()
    if root is not None and (root / "src" / "backend" / "cpu_backend.cpp").exists():
        subprocess.run(["make", "-s", "-C", str(HERE), "ref", f"HALO_REF_ROOT={root}"], check=True)


def _ptr(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Oracle:
    """The plain-C restatement (halo_oracle.c)."""

    kind = "port"

    def __init__(self) -> None:
        if not ORACLE_SO.exists():
            build()
        L = C.CDLL(str(ORACLE_SO))
        L.halo_oracle_fp16_to_fp32.restype = C.c_float
        L.halo_oracle_fp16_to_fp32.argtypes = [C.c_uint16]
        L.halo_oracle_fp32_to_fp16.restype = C.c_uint16
        L.halo_oracle_fp32_to_fp16.argtypes = [C.c_float]
        L.halo_oracle_row_bytes.restype = C.c_int64
        L.halo_oracle_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.halo_oracle_dequantize_row.restype = C.c_int
        L.halo_oracle_dequantize_row.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        L.halo_oracle_dot.restype = C.c_float
        L.halo_oracle_dot.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.halo_oracle_vec_dot_row.restype = C.c_int
        L.halo_oracle_vec_dot_row.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(C.c_float)]
        L.halo_oracle_gemv.restype = C.c_int
        L.halo_oracle_gemv.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64,
                                       C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]
        L.halo_oracle_lm_head.restype = C.c_int
        L.halo_oracle_lm_head.argtypes = [C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64,
                                          C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]
        self.L = L

    def default_threads(self) -> int:
        return os.cpu_count() or 1

    def fp16_to_fp32(self, h: int) -> float:
        return float(self.L.halo_oracle_fp16_to_fp32(h))

    def fp32_to_fp16(self, f: float) -> int:
        return int(self.L.halo_oracle_fp32_to_fp16(f))

    def row_bytes(self, wtype: int, n: int) -> int:
        return int(self.L.halo_oracle_row_bytes(wtype, n))

    def dequantize(self, wtype: int, src: np.ndarray, n: int) -> np.ndarray:
        src = np.ascontiguousarray(src).view(np.uint8)
        out = np.empty(n, np.float32)
        rc = self.L.halo_oracle_dequantize_row(wtype, _ptr(src), _ptr(out), n)
        if rc != 0:
            raise ValueError(f"oracle dequantize_row: status {rc}")
        return out

    def dot(self, a: np.ndarray, b: np.ndarray) -> np.float32:
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        return np.float32(self.L.halo_oracle_dot(_ptr(a), _ptr(b), a.size))

    def vec_dot_row(self, wtype: int, row: np.ndarray, x: np.ndarray) -> np.float32:
        out = C.c_float()
        rc = self.L.halo_oracle_vec_dot_row(wtype, _ptr(np.ascontiguousarray(row)), _ptr(np.ascontiguousarray(x, np.float32)),
                                            x.size, C.byref(out))
        if rc != 0:
            raise ValueError(f"oracle vec_dot_row: status {rc}")
        return np.float32(out.value)

    def gemv(self, wtype: int, w: np.ndarray, x: np.ndarray, rows: int, cols: int, *, w_stride: int = 0,
             threads: int | None = None, status: bool = False):
        """x: [n_vec, cols] fp32 (C-contiguous); returns y [n_vec, rows] fp32."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, cols) if cols else np.zeros((x.shape[0], 0), np.float32)
        n_vec = x.shape[0]
        y = np.zeros((n_vec, rows), np.float32)
        rc = self.L.halo_oracle_gemv(wtype, _ptr(np.ascontiguousarray(w)), w_stride, _ptr(x), 0, _ptr(y), 0, rows, cols, n_vec,
                                     threads or self.default_threads())
        if status:
            return rc, y
        if rc != 0:
            raise ValueError(f"oracle gemv: status {rc}")
        return y

    def lm_head(self, wtype: int, w: np.ndarray, x: np.ndarray, rows: int, cols: int, *, valid_rows: int = 0,
                want_logits: bool = True, want_ids: bool = True, threads: int | None = None):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
        n_vec = x.shape[0]
        logits = np.zeros((n_vec, rows), np.float32) if want_logits else None
        result = np.zeros((n_vec, 3), np.uint32)
        ids = np.zeros(n_vec, np.int32) if want_ids else None
        rc = self.L.halo_oracle_lm_head(wtype, _ptr(np.ascontiguousarray(w)), 0, _ptr(x), 0, _ptr(logits), 0, _ptr(result),
                                        _ptr(ids), rows, cols, n_vec, valid_rows, threads or self.default_threads())
        if rc != 0:
            raise ValueError(f"oracle lm_head: status {rc}")
        return result, logits, ids


class Reference:
    """The unmodified reference CPU backend behind its own Backend interface."""

    kind = "reference"

    @staticmethod
    def available() -> bool:
        return REF_SO.exists()

    def __init__(self, threads: int | None = None) -> None:
        if not REF_SO.exists():
            raise FileNotFoundError(f"{REF_SO} was not built (needs the reference tree at build time)")
        L = C.CDLL(str(REF_SO))
        L.halo_ref_last_error.restype = C.c_char_p
        L.halo_ref_default_threads.restype = C.c_int
        L.halo_ref_fp16_to_fp32.restype = C.c_float
        L.halo_ref_fp16_to_fp32.argtypes = [C.c_uint16]
        L.halo_ref_fp32_to_fp16.restype = C.c_uint16
        L.halo_ref_fp32_to_fp16.argtypes = [C.c_float]
        L.halo_ref_row_bytes.restype = C.c_int64
        L.halo_ref_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.halo_ref_dequantize_row.restype = C.c_int
        L.halo_ref_dequantize_row.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        L.halo_ref_session_create.restype = C.c_void_p
        L.halo_ref_session_create.argtypes = [C.c_int]
        L.halo_ref_session_destroy.argtypes = [C.c_void_p]
        L.halo_ref_gemv.restype = C.c_int
        L.halo_ref_gemv.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64] * 3 + \
            [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
        L.halo_ref_lm_head.restype = C.c_int
        L.halo_ref_lm_head.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_uint64,
                                       C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_uint32,
                                       C.c_uint32, C.c_uint32, C.c_uint32]
        self.L = L
        self.threads = threads or int(L.halo_ref_default_threads())
        self.session = C.c_void_p(L.halo_ref_session_create(self.threads))

    def __del__(self) -> None:
        try:
            if getattr(self, "session", None):
                self.L.halo_ref_session_destroy(self.session)
                self.session = None
        except Exception:
            pass

    def default_threads(self) -> int:
        return self.threads

    def last_error(self) -> str:
        return (self.L.halo_ref_last_error() or b"").decode()

    def fp16_to_fp32(self, h: int) -> float:
        return float(self.L.halo_ref_fp16_to_fp32(h))

    def fp32_to_fp16(self, f: float) -> int:
        return int(self.L.halo_ref_fp32_to_fp16(f))

    def row_bytes(self, wtype: int, n: int) -> int:
        return int(self.L.halo_ref_row_bytes(wtype, n))

    def dequantize(self, wtype: int, src: np.ndarray, n: int) -> np.ndarray:
        src = np.ascontiguousarray(src).view(np.uint8)
        out = np.empty(n, np.float32)
        rc = self.L.halo_ref_dequantize_row(wtype, _ptr(src), _ptr(out), n)
        if rc != 0:
            raise ValueError(f"reference dequantize_row: status {rc}: {self.last_error()}")
        return out

    def gemv_raw(self, wtype: int, w: np.ndarray, x: np.ndarray, y: np.ndarray, rows: int, cols: int, n_vec: int, *,
                 w_off: int = 0, w_stride: int = 0, x_off: int = 0, x_stride: int = 0, y_off: int = 0, y_stride: int = 0,
                 variant_id: int = 0) -> int:
        """The Backend::gemv call on three host arrays with TensorRef-style offsets / strides (bytes)."""
        return int(self.L.halo_ref_gemv(self.session, wtype, _ptr(w), w.nbytes, w_off, w_stride, _ptr(x), x.nbytes, x_off,
                                        x_stride, _ptr(y), y.nbytes, y_off, y_stride, rows, cols, n_vec, variant_id))

    def gemv(self, wtype: int, w: np.ndarray, x: np.ndarray, rows: int, cols: int, *, w_stride: int = 0,
             threads: int | None = None):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
        n_vec = x.shape[0]
        y = np.zeros((n_vec, rows), np.float32)
        w = np.ascontiguousarray(w)
        rc = self.gemv_raw(wtype, w, x, y, rows, cols, n_vec, w_stride=w_stride)
        if rc != 0:
            raise ValueError(f"reference gemv: status {rc}: {self.last_error()}")
        return y

    def lm_head(self, wtype: int, w: np.ndarray, x: np.ndarray, rows: int, cols: int, *, valid_rows: int = 0,
                want_logits: bool = True, want_ids: bool = True, threads: int | None = None):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
        n_vec = x.shape[0]
        w = np.ascontiguousarray(w)
        logits = np.zeros((n_vec, rows), np.float32) if want_logits else None
        result = np.zeros((n_vec, 3), np.uint32)
        ids = np.zeros(n_vec, np.int32) if want_ids else None
        rc = self.L.halo_ref_lm_head(self.session, wtype, _ptr(w), w.nbytes, 0, _ptr(x), x.nbytes, 0, _ptr(logits),
                                     0 if logits is None else logits.nbytes, 0, _ptr(result), _ptr(ids), rows, cols, n_vec,
                                     valid_rows)
        if rc != 0:
            raise ValueError(f"reference lm_head: status {rc}: {self.last_error()}")
        return result, logits, ids


def best_checker(threads: int | None = None):
    """The compiled reference when it was built, else the C restatement."""
    return Reference(threads) if Reference.available() else Oracle()
