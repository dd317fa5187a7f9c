"""The C-ABI library loads and exports every symbol the headers under include/ declare.  CPU only: no compute calls."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import pytest

from halo_b200 import capi

HEADERS = sorted((Path(__file__).resolve().parents[1] / "include").glob("*.h"))


def declared_functions() -> list[str]:
    text = "\n".join(h.read_text() for h in HEADERS)
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(halo_(?:cuda|gguf)_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_in_tree():
    assert capi.LIB_PATH.exists(), "run python -m halo_b200.build"
    assert capi.LIB_PATH.parent.name == "halo_b200"


def test_every_declared_symbol_is_exported_and_bound():
    lib = capi.load()
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared under include/ but not exported"
        assert n in capi.SYMBOLS, f"{n} has no ctypes prototype"
    assert sorted(capi.SYMBOLS) == names


def test_geometry_and_registry_need_no_device():
    lib = capi.load()
    out = C.c_uint64()
    assert lib.halo_cuda_row_bytes(12, 5120, C.byref(out)) == 0 and out.value == 2880
    assert lib.halo_cuda_row_bytes(14, 17408, C.byref(out)) == 0 and out.value == 14280
    assert lib.halo_cuda_row_bytes(8, 17408, C.byref(out)) == 0 and out.value == 18496
    assert lib.halo_cuda_row_bytes(2, 5120, C.byref(out)) == 0 and out.value == 2880
    assert lib.halo_cuda_row_bytes(12, 100, C.byref(out)) == capi.E_MODEL
    assert lib.halo_cuda_row_bytes(5, 32, C.byref(out)) == capi.E_UNSUPPORTED
    assert "block size" in capi.last_error() or "type" in capi.last_error()
    # the id -> name map is append-only and pinned (include/halo/backend/backend.h:210-216)
    arr = (capi.Variant * 16)()
    n = C.c_uint32()
    assert lib.halo_cuda_variants(capi.OP_GEMV, arr, 16, C.byref(n)) == 0
    got = {arr[i].id: arr[i].name.decode() for i in range(n.value)}
    assert got == {1: "gemv_exact8", 2: "gemv_warp_f32", 3: "gemv_mma_f16x2", 4: "gemm_tcgen05_f16", 5: "gemm_tcgen05_bf16",
                   6: "gemv_mma_m1", 7: "gemv_mma_r", 8: "gemv_mma_i8x2", 9: "gemv_mma_i8x2_r", 10: "gemm_tcgen05_f16_r", 11: "gemm_tcgen05_bf16_r"}
    assert lib.halo_cuda_variants(1, arr, 16, C.byref(n)) == capi.E_UNSUPPORTED  # RMS_NORM is not this backend's


def test_no_device_means_failure_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    lib = capi.load()
    ctx = C.c_void_p()
    assert lib.halo_cuda_ctx_create(0, C.byref(ctx)) == capi.E_DEVICE
    assert not ctx.value


def test_product_does_not_import_the_oracle():
    pkg = Path(capi.__file__).resolve().parent
    for p in list(pkg.rglob("*.py")) + list(pkg.rglob("*.cu")) + list(pkg.rglob("*.cpp")) + list(pkg.rglob("*.h")):
        text = p.read_text()
        assert "import oracle" not in text and "from oracle" not in text and "liboracle" not in text, p
