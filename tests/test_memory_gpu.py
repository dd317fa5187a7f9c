"""Device memory of the C ABI: blocks come from a per-context pool (the model allocates every activation buffer of a forward
through Backend::allocate, src/models/qwen35.cpp:462-465), stay zero-filled on reuse, and shareable blocks stay exportable."""
from __future__ import annotations

import ctypes as C
import time

import numpy as np
import pytest

from halo_b200 import backend as hb
from halo_b200 import capi

pytestmark = pytest.mark.gpu


def test_reused_blocks_are_zero_filled_and_cheap():
    be = hb.CudaBackend(0)
    st = be.create_stream()
    n = 1 << 20
    seen = set()
    for i in range(8):
        b = be.allocate(n)
        got = np.empty(n, np.uint8)
        be.download(st, hb.TensorRef.of(b), got)
        st.wait()
        assert not got.any(), f"allocation {i} is not zero-filled"
        be.upload(st, hb.TensorRef.of(b), np.full(n, 0xA5, np.uint8))
        st.wait()
        seen.add(b.ptr)
        b.free()
    assert len(seen) < 8, "freed blocks are never handed out again: the pool is not in use"
    # not a benchmark, only a guard against a driver call per allocation: a pool hit costs microseconds
    t0 = time.perf_counter()
    for _ in range(200):
        be.allocate(4096).free()
    per_pair = (time.perf_counter() - t0) / 200
    assert per_pair < 200e-6, f"allocate + free took {per_pair * 1e6:.0f} us"


def test_pool_blocks_cannot_be_exported_but_shareable_ones_can():
    be = hb.CudaBackend(0)
    h = C.create_string_buffer(64)
    pooled = be.allocate(4096)
    assert be.lib.halo_cuda_ipc_export(be.ctx, C.c_void_p(pooled.ptr), h) == capi.E_KERNEL
    assert "SHAREABLE" in capi.last_error()
    shared = be.allocate(4096, shareable=True)
    assert be.lib.halo_cuda_ipc_export(be.ctx, C.c_void_p(shared.ptr), h) == 0
    st = be.create_stream()
    got = np.ones(4096, np.uint8)
    be.download(st, hb.TensorRef.of(shared), got)
    st.wait()
    assert not got.any()
