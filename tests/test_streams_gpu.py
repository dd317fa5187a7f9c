"""Several streams on one context (Backend::create_stream hands out any number, include/halo/backend/backend.h:494-506): calls on
different streams may overlap on the device, so nothing they use may be shared between them.  The kernels' on-demand scratch
(row-block counters, cross-CTA partial sums, staged activations, LM-head partials) is kept per stream; this test interleaves
calls that use all of it on two streams without waiting in between and expects the single-stream bits."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits
from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu


def test_two_streams_do_not_share_scratch():
    be = hb.CudaBackend(0)
    s1, s2 = be.create_stream(), be.create_stream()
    cases = [(synth.Q4_K, 2176, 5120, 1, 0),   # row blocks shared between CTAs: counters and partial sums
             (synth.Q4_K, 640, 2560, 5, 0),     # a batch: activations staged in scratch by a kernel of their own
             (synth.Q4_K, 2176, 5120, 3, capi.GEMV_MMA_F16X2)]
    ops = []
    for i, (t, n, k, m, v) in enumerate(cases):
        w = synth.quant_weights(t, n, k, 50 + i, 1)
        x = synth.activations(m, k, 50 + i, 2)
        wb, xb = be.import_host_readonly(w.reshape(-1)), be.import_host_readonly(x)
        ya, yb = be.allocate(m * n * 4), be.allocate(m * n * 4)
        ops.append((hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(ya), n, k, m, v),
                    hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m, v), m, n))
    s1.wait()
    # the single-stream answers
    want = []
    for a, _, m, n in ops:
        be.gemv(s1, a)
        y = np.empty((m, n), np.float32)
        be.download(s1, a.y, y)
        s1.wait()
        want.append(y)
    # interleaved on two streams, many times, no waits in between
    for _ in range(30):
        for a, b, _, _ in ops:
            be.gemv(s1, a)
            be.gemv(s2, b)
    got = []
    for a, b, m, n in ops:
        ya, yb = np.empty((m, n), np.float32), np.empty((m, n), np.float32)
        be.download(s1, a.y, ya)
        be.download(s2, b.y, yb)
        got.append((ya, yb))
    s1.wait()
    s2.wait()
    for (ya, yb), y in zip(got, want):
        assert np.array_equal(bits(ya), bits(y)) and np.array_equal(bits(yb), bits(y))
    assert be.scratch_bytes() > 0


def test_two_devices_in_one_process_each_raise_their_own_kernel_attributes():
    """A kernel's opt-in to large dynamic shared memory is a per-device attribute: a second context on another device must set it
    again for itself (a process-wide "already done" flag would leave the second device's launches refused)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    t, n, k = synth.Q4_K, 2176, 5120
    w = synth.quant_weights(t, n, k, 60, 1)
    x = synth.activations(20, k, 60, 2)
    ys = []
    for dev in (0, 1):
        be = hb.CudaBackend(dev)
        st = be.create_stream()
        wb, xb = be.import_host_readonly(w.reshape(-1)), be.import_host_readonly(x)
        got = []
        for m, variant, gemm in ((1, 0, False), (5, 0, False), (3, capi.GEMV_MMA_F16X2, False), (20, capi.GEMM_TCGEN05_F16, True)):
            yb = be.allocate(m * n * 4)
            be.gemv(st, hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m, variant, allow_gemm=gemm))
            y = np.empty((m, n), np.float32)
            be.download(st, hb.TensorRef.of(yb), y)
            st.wait()
            got.append(y)
        ys.append(got)
    for a, b in zip(*ys):
        assert np.array_equal(bits(a), bits(b)), "the two devices run the same kernels on the same bytes"
