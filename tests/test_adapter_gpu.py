"""The C++ adapter (halo::backend::Backend over the C ABI) against the unmodified reference CPU backend, both called
through the reference's own interface by tests/native/adapter_selftest.cpp."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
SELFTEST = ROOT / "tests" / "native" / "libadapter_selftest.so"
ADAPTER = ROOT / "halo_b200" / "adapter" / "libhalo_cuda_backend.so"


def test_adapter_library_exports_the_factory():
    if not ADAPTER.exists():
        pytest.skip("the adapter was not built (needs the reference headers at build time)")
    data = ADAPTER.read_bytes()
    assert b"make_cuda_backend" in data and b"cuda_backend_set_plan" in data
    assert b"halo_oracle" not in data and b"libhalo_ref" not in data  # the product does not link the checker


@pytest.mark.gpu
def test_adapter_against_reference_cpu_backend_through_the_interface():
    if not SELFTEST.exists():
        pytest.skip("the native selftest was not built (needs the reference tree at build time)")
    lib = C.CDLL(str(SELFTEST))
    lib.halo_adapter_selftest.restype = C.c_int
    lib.halo_adapter_selftest.argtypes = [C.c_char_p, C.c_size_t]
    buf = C.create_string_buffer(16384)
    failed = lib.halo_adapter_selftest(buf, len(buf))
    report = buf.value.decode(errors="replace")
    assert failed == 0, report
    assert "checks passed" in report
