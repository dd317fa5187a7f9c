"""The allocation-free LM head entry point against the regular one, through the C ABI.

Some hosts size every device buffer when they start and must not call the allocator afterwards (a latency-bound
serving loop, an embedder with a fixed memory budget).  halo_cuda_lm_head_noalloc serves them: its argmax partials
live in a fixed array of the library instead of context scratch that grows on demand.  The file name sorts last on
purpose: a run that stops at the first failure has then already run every other test."""
from __future__ import annotations

import numpy as np
import pytest

from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu


def _run(be, st, entry, wtype, w, x, rows, cols, valid_rows=0, variant=0, no_scratch=False):
    n_vec = x.shape[0]
    wb = be.import_host_readonly(w.reshape(-1))
    xb = be.import_host_readonly(x)
    lb = be.allocate(n_vec * rows * 4)
    rb = be.allocate(n_vec * 12)
    ib = be.allocate(n_vec * 4)
    g = hb.GemvArgs(wtype, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(lb), rows, cols, n_vec, variant, no_scratch=no_scratch)
    a = hb.LmHeadArgs(g, hb.TensorRef.of(rb), valid_rows, hb.TensorRef.of(ib))
    entry(st, a)
    res = np.zeros((n_vec, 3), np.uint32)
    logits = np.zeros((n_vec, rows), np.float32)
    ids = np.zeros(n_vec, np.int32)
    be.download(st, hb.TensorRef.of(rb), res)
    be.download(st, hb.TensorRef.of(lb), logits)
    be.download(st, hb.TensorRef.of(ib), ids)
    st.wait()
    return res, logits, ids


def test_noalloc_lm_head_equals_regular_lm_head_twice_in_a_row():
    be = hb.CudaBackend(0)
    st = be.create_stream()
    # two different calls back to back: the second must not be disturbed by what the first left in the shared scratch
    cases = [(synth.Q4_K, 8192 + 900, 512, 3, 0, 0), (synth.Q8_0, 20000, 256, 16, 15000, capi.GEMV_EXACT8)]
    for wtype, rows, cols, n_vec, valid, variant in cases:
        w = synth.quant_weights(wtype, rows, cols, 91 + wtype, 1)
        x = synth.activations(n_vec, cols, 91 + wtype, 2)
        x[n_vec - 1, 3] = np.nan  # one poisoned vector: the NaN flag travels through the partials too
        # the regular entry point under the no-scratch flag takes the kernels the allocation-free one is limited to
        want = _run(be, st, be.lm_head, wtype, w, x, rows, cols, valid, variant, no_scratch=True)
        got = _run(be, st, be.lm_head_noalloc, wtype, w, x, rows, cols, valid, variant)
        # same kernels, same order of operations: bit-identical words, logits and ids (the suite's bar for integer work)
        assert np.array_equal(got[0], want[0])
        assert np.array_equal(got[1].view(np.uint32), want[1].view(np.uint32))
        assert np.array_equal(got[2], want[2])
        assert got[0][n_vec - 1, 2] == 1 and got[2][n_vec - 1] == 0
        # and the default kernels (context scratch allowed) agree with it to their own rounding: same ids, logits within 2e-4 of the
        # largest (Q4_K's default is the int8 family, 16-bit fixed-point x) or 1e-5 (a kernel named by the caller)
        free = _run(be, st, be.lm_head, wtype, w, x, rows, cols, valid, variant)
        ok = np.isfinite(want[1])
        assert np.array_equal(free[2], want[2])
        assert np.max(np.abs(free[1][ok] - want[1][ok])) <= (2e-4 if variant == 0 else 1e-5) * np.max(np.abs(want[1][ok]))


def test_noalloc_lm_head_rejects_what_does_not_fit_and_needs_a_logits_buffer():
    be = hb.CudaBackend(0)
    st = be.create_stream()
    rows, cols, n_vec = 8192 * 300, 32, 16  # 300 chunks x 16 vectors = 4800 partial records > 4096
    wb = be.allocate(64)  # never read: the call must be refused before anything is enqueued
    xb = be.allocate(n_vec * cols * 4)
    rb = be.allocate(n_vec * 12)
    g = hb.GemvArgs(synth.Q8_0, hb.TensorRef(wb, 0, 0, 0), hb.TensorRef.of(xb), hb.TensorRef(), rows, cols, n_vec, 0)
    a = hb.LmHeadArgs(g, hb.TensorRef.of(rb))
    with pytest.raises(hb.HaloError):  # no logits buffer
        be.lm_head_noalloc(st, a)
    import ctypes as C
    h = capi.LmHead()
    h.gemv.wtype, h.gemv.rows, h.gemv.cols, h.gemv.n_vec = synth.Q8_0, rows, cols, n_vec
    h.gemv.w, h.gemv.x, h.gemv.y = 0x1000000, xb.ptr, 0x2000000000  # placeholders: validation happens on the host only
    h.result = rb.ptr
    rc = be.lib.halo_cuda_lm_head_noalloc(be.ctx, C.byref(h), st.handle)
    assert rc == capi.E_UNSUPPORTED
    assert "fixed scratch" in capi.last_error()
    st.wait()


def test_noalloc_lm_head_takes_no_context_scratch_and_checks_aliases_like_the_regular_one():
    """On a context of its own the allocation-free entry point leaves the context's on-demand scratch at zero bytes, where the
    regular one grows it; and it refuses outputs that overlap an operand with the same error class."""
    import ctypes as C
    be = hb.CudaBackend(0)
    st = be.create_stream()
    wtype, rows, cols, n_vec = synth.Q4_K, 9000, 512, 3
    w = synth.quant_weights(wtype, rows, cols, 17, 1)
    x = synth.activations(n_vec, cols, 17, 2)
    assert be.scratch_bytes() == 0
    got = _run(be, st, be.lm_head_noalloc, wtype, w, x, rows, cols)
    assert be.scratch_bytes() == 0, "the allocation-free LM head grew context scratch"
    want = _run(be, st, be.lm_head, wtype, w, x, rows, cols, no_scratch=True)  # same kernels through the regular entry point
    assert be.scratch_bytes() > 0  # ... which keeps its logits / argmax partials in context scratch
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[2], want[2])
    # aliasing: result inside the logits buffer, ids inside x -- refused before anything is enqueued, by both entry points
    wb = be.import_host_readonly(w.reshape(-1))
    xb = be.import_host_readonly(x)
    lb = be.allocate(n_vec * rows * 4)
    rb = be.allocate(n_vec * 12)
    for entry in (be.lib.halo_cuda_lm_head_noalloc, be.lib.halo_cuda_lm_head):
        for result, ids in ((lb.ptr + 64, None), (rb.ptr, xb.ptr), (rb.ptr, rb.ptr + 4)):
            h = capi.LmHead()
            h.gemv.wtype, h.gemv.rows, h.gemv.cols, h.gemv.n_vec = wtype, rows, cols, n_vec
            h.gemv.w, h.gemv.x, h.gemv.y = wb.ptr, xb.ptr, lb.ptr
            h.result, h.ids = result, ids
            assert entry(be.ctx, C.byref(h), st.handle) == capi.E_KERNEL, capi.last_error()
            assert "overlaps" in capi.last_error()
    st.wait()
