"""ctypes binding of libhalo_cuda.so (the C ABI declared in include/halo_cuda.h and include/halo_cuda_gguf.h).

The library is the product; this module only loads it and mirrors its structs.  There is no CPU
fallback: if the library is missing, or no sm_100 device is present, the calls fail loudly.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libhalo_cuda.so"

OK = 0
E_MODEL, E_MEMORY, E_BACKEND, E_KERNEL, E_CONFIG, E_API, E_DEVICE, E_UNSUPPORTED, E_IO = -1, -2, -3, -4, -5, -6, -7, -8, -9
ERROR_NAMES = {E_MODEL: "Model", E_MEMORY: "Memory", E_BACKEND: "Backend", E_KERNEL: "Kernel", E_CONFIG: "Config", E_API: "Api",
               E_DEVICE: "Device", E_UNSUPPORTED: "Unsupported", E_IO: "Io"}
SPLIT_NONE, SPLIT_COLUMN, SPLIT_ROW = 0, 1, 2

OP_GET_ROWS, OP_GEMV, OP_LM_HEAD = 0, 3, 14
GEMV_DEFAULT, GEMV_EXACT8, GEMV_WARP_F32, GEMV_MMA_F16X2, GEMM_TCGEN05_F16, GEMM_TCGEN05_BF16, GEMV_MMA_M1, GEMV_MMA_R = 0, 1, 2, 3, 4, 5, 6, 7
GEMV_MMA_I8X2 = 8
GEMV_MMA_I8X2_R = 9
GEMM_TCGEN05_F16_R, GEMM_TCGEN05_BF16_R = 10, 11
REPACKED_VARIANTS = (GEMV_MMA_R, GEMV_MMA_I8X2_R, GEMM_TCGEN05_F16_R, GEMM_TCGEN05_BF16_R)  # W is in the layout of halo_cuda_repack_rows
FLAG_ALLOW_GEMM = 1
FLAG_NO_SCRATCH = 0x80000000


class DeviceInfo(C.Structure):
    _fields_ = [("name", C.c_char * 128), ("pci_id", C.c_char * 16), ("arch", C.c_char * 16), ("cc_major", C.c_int32),
                ("cc_minor", C.c_int32), ("sm_count", C.c_int32), ("l2_bytes", C.c_int32), ("driver_version", C.c_int32),
                ("runtime_version", C.c_int32), ("total_bytes", C.c_uint64), ("clock_khz", C.c_int32), ("mem_clock_khz", C.c_int32)]


class Variant(C.Structure):
    _fields_ = [("id", C.c_uint32), ("op", C.c_uint32), ("family", C.c_uint32), ("name", C.c_char_p)]


class Gemv(C.Structure):
    _fields_ = [("wtype", C.c_uint32), ("variant_id", C.c_uint32), ("w", C.c_void_p), ("w_stride", C.c_uint64), ("x", C.c_void_p),
                ("x_stride", C.c_uint64), ("y", C.c_void_p), ("y_stride", C.c_uint64), ("rows", C.c_uint32), ("cols", C.c_uint32),
                ("n_vec", C.c_uint32), ("flags", C.c_uint32)]


class GemvPlan(C.Structure):
    _fields_ = [("slices", C.c_uint32), ("ctas", C.c_uint32), ("cols_per_unit", C.c_uint32), ("reserved", C.c_uint32),
                ("start", C.c_uint32 * 161)]


class GemvTiles(C.Structure):
    _fields_ = [("tile_rows", C.c_uint32), ("launches", C.c_uint32), ("conversions", C.c_uint32), ("streamed", C.c_uint32),
                ("stretch_cols", C.c_uint32), ("resident_rows", C.c_uint32), ("reserved", C.c_uint32 * 2)]


class PeerReduce(C.Structure):
    _fields_ = [("world", C.c_uint32), ("rank", C.c_uint32), ("capacity", C.c_uint32), ("reserved", C.c_uint32),
                ("slots", C.c_void_p * 8), ("epoch", C.c_void_p), ("done", C.c_void_p)]


class LmHead(C.Structure):
    _fields_ = [("gemv", Gemv), ("result", C.c_void_p), ("ids", C.c_void_p), ("valid_rows", C.c_uint32), ("row_offset", C.c_uint32)]


class GetRows(C.Structure):
    _fields_ = [("type", C.c_uint32), ("variant_id", C.c_uint32), ("table", C.c_void_p), ("table_stride", C.c_uint64),
                ("ids", C.c_void_p), ("out", C.c_void_p), ("out_stride", C.c_uint64), ("n_rows", C.c_uint32), ("cols", C.c_uint32),
                ("n_ids", C.c_uint32), ("status", C.c_void_p)]


class GgufInfo(C.Structure):
    _fields_ = [("version", C.c_uint32), ("alignment", C.c_uint32), ("n_kv", C.c_uint64), ("n_tensors", C.c_uint64),
                ("header_size", C.c_uint64), ("data_offset", C.c_uint64), ("file_size", C.c_uint64)]


class GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("n_dims", C.c_uint32), ("type", C.c_uint32), ("ne", C.c_int64 * 4), ("offset", C.c_uint64),
                ("n_elements", C.c_uint64), ("n_bytes", C.c_uint64), ("supported", C.c_uint32), ("reserved", C.c_uint32)]


class Upload(C.Structure):
    _fields_ = [("split", C.c_uint32), ("rank", C.c_uint32), ("world", C.c_uint32), ("repack", C.c_uint32), ("staging_bytes", C.c_uint64)]


class Matrix(C.Structure):
    _fields_ = [("w", C.c_void_p), ("w_stride", C.c_uint64), ("bytes", C.c_uint64), ("wtype", C.c_uint32), ("variant_id", C.c_uint32),
                ("rows", C.c_uint32), ("cols", C.c_uint32), ("row0", C.c_uint32), ("k0", C.c_uint32)]


# Every symbol the two headers declare: name -> (restype, argtypes)
_P = C.c_void_p
SYMBOLS = {
    "halo_cuda_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "halo_cuda_ctx_create": (C.c_int, [C.c_int, C.POINTER(_P)]),
    "halo_cuda_ctx_destroy": (C.c_int, [_P]),
    "halo_cuda_device_info": (C.c_int, [_P, C.POINTER(DeviceInfo)]),
    "halo_cuda_malloc": (C.c_int, [_P, C.c_uint64, C.c_int, C.POINTER(_P)]),
    "halo_cuda_free": (C.c_int, [_P, _P]),
    "halo_cuda_stream_create": (C.c_int, [_P, C.POINTER(_P)]),
    "halo_cuda_stream_destroy": (C.c_int, [_P, _P]),
    "halo_cuda_stream_sync": (C.c_int, [_P, _P, C.c_uint64]),
    "halo_cuda_ctx_lost": (C.c_int, [_P]),
    "halo_cuda_ctx_set_peer_wait_polls": (C.c_int, [_P, C.c_uint32]),
    "halo_cuda_ctx_scratch_bytes": (C.c_int, [_P, C.POINTER(C.c_uint64)]),
    "halo_cuda_memcpy_h2d_async": (C.c_int, [_P, _P, _P, C.c_uint64, _P]),
    "halo_cuda_memcpy_d2h_async": (C.c_int, [_P, _P, _P, C.c_uint64, _P]),
    "halo_cuda_memcpy_d2d_async": (C.c_int, [_P, _P, _P, C.c_uint64, _P]),
    "halo_cuda_memset_async": (C.c_int, [_P, _P, C.c_int, C.c_uint64, _P]),
    "halo_cuda_host_alloc": (C.c_int, [_P, C.c_uint64, C.POINTER(_P)]),
    "halo_cuda_host_free": (C.c_int, [_P, _P]),
    "halo_cuda_event_create": (C.c_int, [_P, C.POINTER(_P)]),
    "halo_cuda_event_destroy": (C.c_int, [_P, _P]),
    "halo_cuda_event_record": (C.c_int, [_P, _P, _P]),
    "halo_cuda_event_elapsed_ns": (C.c_int, [_P, _P, _P, C.POINTER(C.c_uint64)]),
    "halo_cuda_row_bytes": (C.c_int, [C.c_uint32, C.c_uint64, C.POINTER(C.c_uint64)]),
    "halo_cuda_variants": (C.c_int, [C.c_uint32, C.POINTER(Variant), C.c_uint32, C.POINTER(C.c_uint32)]),
    "halo_cuda_gemv_resolve": (C.c_int, [_P, C.POINTER(Gemv), C.POINTER(C.c_uint32)]),
    "halo_cuda_plan_set": (C.c_int, [_P, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "halo_cuda_plan_clear": (C.c_int, [_P]),
    "halo_cuda_last_error": (C.c_size_t, [C.c_char_p, C.c_size_t]),
    "halo_cuda_gemv": (C.c_int, [_P, C.POINTER(Gemv), _P]),
    "halo_cuda_gemv_normed": (C.c_int, [_P, C.POINTER(Gemv), _P, C.c_float, _P]),
    "halo_cuda_gemv_gated": (C.c_int, [_P, C.POINTER(Gemv), _P, _P, C.c_uint32, _P]),
    "halo_cuda_lm_head": (C.c_int, [_P, C.POINTER(LmHead), _P]),
    "halo_cuda_get_rows": (C.c_int, [_P, C.POINTER(GetRows), _P]),
    "halo_cuda_lm_head_noalloc": (C.c_int, [_P, C.POINTER(LmHead), _P]),
    "halo_cuda_repacked_row_bytes": (C.c_int, [C.c_uint32, C.c_uint64, C.POINTER(C.c_uint64)]),
    "halo_cuda_gemv_plan_i8": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(GemvPlan)]),
    "halo_cuda_gemv_tiles_i8": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(GemvTiles)]),
    "halo_cuda_repacked_variant": (C.c_int, [C.c_uint32, C.c_uint64, C.POINTER(C.c_uint32)]),
    "halo_cuda_repack_rows": (C.c_int, [_P, C.c_uint32, _P, C.c_uint64, _P, C.c_uint64, C.c_uint32, C.c_uint32, _P]),
    "halo_cuda_gemv_plan": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(GemvPlan)]),
    "halo_cuda_ipc_export": (C.c_int, [_P, _P, C.c_char_p]),
    "halo_cuda_ipc_open": (C.c_int, [_P, C.c_char_p, C.POINTER(_P)]),
    "halo_cuda_ipc_close": (C.c_int, [_P, _P]),
    "halo_cuda_gemv_reduce": (C.c_int, [_P, C.POINTER(Gemv), C.POINTER(PeerReduce), _P]),
    "halo_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(_P)]),
    "halo_gguf_parse": (C.c_int, [_P, C.c_uint64, C.POINTER(_P)]),
    "halo_gguf_close": (C.c_int, [_P]),
    "halo_gguf_info": (C.c_int, [_P, C.POINTER(GgufInfo)]),
    "halo_gguf_kv_u64": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_uint64), C.POINTER(C.c_int)]),
    "halo_gguf_kv_i64": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_int64), C.POINTER(C.c_int)]),
    "halo_gguf_kv_f64": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "halo_gguf_kv_string": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_int)]),
    "halo_gguf_tensor": (C.c_int, [_P, C.c_uint64, C.POINTER(GgufTensor)]),
    "halo_gguf_find": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_uint64), C.POINTER(C.c_int)]),
    "halo_gguf_tensor_data": (C.c_int, [_P, C.c_uint64, C.POINTER(_P), C.POINTER(C.c_uint64)]),
    "halo_cuda_matrix_share": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32, C.POINTER(Upload), C.POINTER(Matrix)]),
    "halo_cuda_upload_matrix": (C.c_int, [_P, _P, C.c_uint64, C.POINTER(Upload), _P, C.POINTER(Matrix)]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the in-tree library and sets every prototype; raises if it was not built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(f"{LIB_PATH} is missing: run `python -m halo_b200.build` (there is no CPU fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(1024)
    load().halo_cuda_last_error(buf, len(buf))
    return buf.value.decode(errors="replace")
