"""Failure detection of the cuda backend, exercised without faulting a GPU.

The reference marks a backend lost when a submission misses its wait budget (Backend::lost(), include/halo/backend/backend.h:517-520)
and injects its failures on the host (tests/unit/runtime/test_engine_faults.cpp:102-357).  Here: a host wait whose budget is far
too short for the work in front of it; the one device-side wait of this backend that depends on another GPU (the adding kernel of
a row split) made to run out by a peer that never writes -- the kernel gives up after its poll limit, raises the context's error
word and stores nothing; and host-side refusals (an allocation nobody can serve, calls on a lost context).  Every case runs on a
context of its own, so that the lost state does not leak into other tests."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu


def test_stream_wait_budget_expiry_marks_the_context_lost():
    be = hb.CudaBackend(0)
    st = be.create_stream()
    t, n, k = synth.Q4_K, 17408, 5120
    wb = be.import_host_readonly(synth.quant_weights(t, n, k, 1, 1).reshape(-1))
    xb = be.import_host_readonly(synth.activations(1, k, 1, 2))
    yb = be.allocate(n * 4)
    a = hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, 1, capi.GEMV_EXACT8)
    st.wait()
    assert not be.lost()
    for _ in range(40):  # about 0.3 ms each on the exact-order kernel: milliseconds of work in front of the wait
        be.gemv(st, a)
    rc = be.lib.halo_cuda_stream_sync(be.ctx, st.handle, 1000)  # a budget of one microsecond
    assert rc == capi.E_BACKEND and "exceeded" in capi.last_error()
    assert be.lost() and be.lib.halo_cuda_ctx_lost(be.ctx) == 1
    # a lost context refuses every later call with Error(Device) and enqueues nothing (include/halo/backend/backend.h:24-26)
    g = be._gemv_struct(a, "MATMUL", False)
    assert be.lib.halo_cuda_gemv(be.ctx, C.byref(g), st.handle) == capi.E_DEVICE
    p = C.c_void_p()
    assert be.lib.halo_cuda_malloc(be.ctx, 4096, 1, C.byref(p)) == capi.E_DEVICE
    assert be.lib.halo_cuda_stream_sync(be.ctx, st.handle, 0) == capi.E_DEVICE
    # the work itself was healthy: destroying the context drains it


def test_row_split_reduction_gives_up_on_a_peer_that_never_writes():
    be = hb.CudaBackend(0)
    st = be.create_stream()
    assert be.lib.halo_cuda_ctx_set_peer_wait_polls(be.ctx, 20000) == 0  # a few milliseconds instead of about a second
    t, n, k = synth.Q4_K, 256, 1024
    wb = be.import_host_readonly(synth.quant_weights(t, n, k, 2, 1).reshape(-1))
    xb = be.import_host_readonly(synth.activations(1, k, 2, 2))
    sentinel = np.full(n, -7.25, np.float32)
    yb = be.allocate(n * 4)
    be.upload(st, hb.TensorRef.of(yb), sentinel)
    capacity = 1024
    mine = be.allocate(2 * 2 * capacity * 8)    # this rank's receive buffer: 2 slot sets x 2 ranks
    silent = be.allocate(2 * 2 * capacity * 8)  # stands in for the peer's buffer: pushed into, never read; and the peer pushes nothing
    words = be.allocate(64)
    st.wait()
    pr = capi.PeerReduce()
    pr.world, pr.rank, pr.capacity = 2, 0, capacity
    pr.slots[0], pr.slots[1] = mine.ptr, silent.ptr
    pr.epoch, pr.done = words.ptr, words.ptr + 16
    g = be._gemv_struct(hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, 1, 0), "MATMUL", False)
    assert be.lib.halo_cuda_gemv_reduce(be.ctx, C.byref(g), C.byref(pr), st.handle) == 0  # enqueued: the loss shows at the wait
    host = np.zeros(n, np.float32)
    be.download(st, hb.TensorRef.of(yb), host)  # behind the kernels in stream order, before the context learns of the loss
    rc = be.lib.halo_cuda_stream_sync(be.ctx, st.handle, 0)
    assert rc == capi.E_BACKEND and "bounded wait" in capi.last_error()
    assert be.lost()
    assert be.lib.halo_cuda_gemv(be.ctx, C.byref(g), st.handle) == capi.E_DEVICE
    # the kernel returned on its own (the device still answers) and stored nothing: y keeps its sentinel
    assert np.array_equal(host, sentinel)
    # another context on the same device is unaffected
    other = hb.CudaBackend(0)
    other.create_stream().wait()
    assert not other.lost()


def test_host_side_refusals_leave_the_context_usable():
    be = hb.CudaBackend(0)
    st = be.create_stream()
    p = C.c_void_p()
    assert be.lib.halo_cuda_malloc(be.ctx, 1 << 50, 1, C.byref(p)) == capi.E_MEMORY  # a petabyte: Error(Memory), nothing changes
    assert not be.lost()
    t, n, k = synth.Q8_0, 64, 256
    wb = be.import_host_readonly(synth.quant_weights(t, n, k, 3, 1).reshape(-1))
    xb = be.import_host_readonly(synth.activations(2, k, 3, 2))
    yb = be.allocate(2 * n * 4)
    be.gemv(st, hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, 2))
    st.wait()
    assert not be.lost()
