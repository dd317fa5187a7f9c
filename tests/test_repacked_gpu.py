"""The repacked-layout tensor-core kernel (gemv_mma_r) for Q6_K / Q8_0 / Q4_0: the repack is a byte permutation
(checked by inverting it on the host), and the products stay within the summation bound of the oracle."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits
from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu
TYPES = (synth.Q6_K, synth.Q8_0, synth.Q4_0)


@pytest.fixture(scope="module")
def be():
    return hb.CudaBackend(0)


def unrepack(wtype: int, packed: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Inverse of halo_cuda_repack_rows on the host, from the documented layout."""
    groups = cols // 256
    if wtype == synth.Q4_0:
        p = packed.reshape(rows, groups, 144)
        raw = np.zeros((rows, groups, 8, 18), np.uint8)
        raw[..., 0:2] = p[..., :16].reshape(rows, groups, 8, 2)
        q = p[..., 16:].reshape(rows, groups, 2, 4, 4, 4)          # chunk, thread, block-in-chunk, byte
        for c in range(2):
            for j in range(4):
                for t in range(4):
                    raw[:, :, 4 * c + j, 2 + 4 * t:6 + 4 * t] = q[:, :, c, t, j]
        return raw.reshape(rows, groups * 144)
    if wtype == synth.Q8_0:
        p = packed.reshape(rows, groups, 272)
        raw = np.zeros((rows, groups, 8, 34), np.uint8)
        raw[..., 0:2] = p[..., :16].reshape(rows, groups, 8, 2)
        q = p[..., 16:].reshape(rows, groups, 4, 4, 4, 4)          # chunk, thread, (parity, step), byte
        for c in range(4):
            for j in range(4):
                for t in range(4):
                    off = 2 + 16 * (j & 1) + 4 * t
                    raw[:, :, 2 * c + (j >> 1), off:off + 4] = q[:, :, c, t, j]
        return raw.reshape(rows, groups * 272)
    p = packed.reshape(rows, groups, 224)
    raw = np.zeros((rows, groups, 210), np.uint8)
    raw[..., 192:208] = p[..., 0:16]
    raw[..., 208:210] = p[..., 16:18]
    ql = p[..., 32:160].reshape(rows, groups, 2, 4, 4, 4)           # half, thread, (b, lh), byte
    qh = p[..., 160:224].reshape(rows, groups, 4, 4, 4)             # thread, (n, lh), byte
    for t in range(4):
        for j in range(4):
            for n in range(2):
                off = 64 * n + 32 * (j >> 1) + 16 * (j & 1) + 4 * t
                raw[..., off:off + 4] = ql[:, :, n, t, j]
            off = 128 + 32 * (j >> 1) + 16 * (j & 1) + 4 * t
            raw[..., off:off + 4] = qh[:, :, t, j]
    return raw.reshape(rows, groups * 210)


def run(be, st, wtype, w, x, rows, cols, offset=0):
    n_vec = x.shape[0]
    buf = np.zeros(offset + w.size, np.uint8)
    buf[offset:] = w.reshape(-1)
    wb = be.import_host_readonly(buf)
    pk = be.repack(st, wtype, hb.TensorRef(wb, offset), rows, cols)
    xb = be.import_host_readonly(x)
    yb = be.allocate(n_vec * rows * 4)
    be.gemv(st, hb.GemvArgs(wtype, hb.TensorRef.of(pk), hb.TensorRef.of(xb), hb.TensorRef.of(yb), rows, cols, n_vec, capi.GEMV_MMA_R))
    y = np.empty((n_vec, rows), np.float32)
    be.download(st, hb.TensorRef.of(yb), y)
    packed = np.empty(rows * be.repacked_row_bytes(wtype, cols), np.uint8)
    be.download(st, hb.TensorRef.of(pk), packed)
    st.wait()
    return y, packed


@pytest.mark.parametrize("t", TYPES)
def test_repack_is_a_byte_permutation(be, t):
    rows, cols = 19, 1024
    w = synth.random_blocks_finite(t, rows, cols, 71, t)
    st = be.create_stream()
    _, packed = run(be, st, t, w, synth.activations(1, cols, 71, 2), rows, cols, offset=3)  # raw rows at an odd byte offset
    assert np.array_equal(unrepack(t, packed, rows, cols), w)
    assert be.repacked_row_bytes(t, cols) == cols // 256 * {synth.Q4_0: 144, synth.Q8_0: 272, synth.Q6_K: 224}[t]
    with pytest.raises(hb.HaloError):
        be.repacked_row_bytes(synth.Q4_K, 1024)
    with pytest.raises(hb.HaloError):
        be.repacked_row_bytes(t, 1000)


@pytest.mark.parametrize("t,n,k,m", [(synth.Q6_K, 5120, 17408, 1), (synth.Q6_K, 5120, 17408, 4), (synth.Q6_K, 5120, 17408, 8),
                                     (synth.Q8_0, 5120, 17408, 1), (synth.Q8_0, 5120, 17408, 8), (synth.Q4_0, 17408, 5120, 16),
                                     (synth.Q6_K, 37, 512, 3), (synth.Q8_0, 130, 256, 21), (synth.Q4_0, 13, 5120, 17), (synth.Q4_0, 1000, 2560, 5),
                                     # more tiles than warps: several passes per warp, sums carried from one pass to the next
                                     (synth.Q4_0, 40000, 256, 2), (synth.Q6_K, 50000, 768, 5), (synth.Q8_0, 60001, 512, 16)])
def test_repacked_kernel_within_summation_bound(be, checker, t, n, k, m):
    from gpu_util import summation_bound
    w = synth.quant_weights(t, n, k, 0, 1)
    x = synth.activations(m, k, 0, 2)
    y, _ = run(be, be.create_stream(), t, w, x, n, k)
    ref = checker.gemv(t, w, x, n, k)
    bound = summation_bound(checker.dequantize, t, w, x, n, k, depth=2 * (k // 8 + 8))
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err <= bound), f"max err/bound {np.max(err / np.maximum(bound, 1e-30)):.3f}"
    assert np.max(err) <= 1e-3 * np.max(np.abs(ref))
    if n * m >= 1000:
        assert not np.array_equal(bits(y), bits(ref))


@pytest.mark.parametrize("t", TYPES)
def test_repacked_kernel_rows_do_not_depend_on_batch_size(be, t):
    n, k = 48, 17408   # K large enough that 1, 4 and 16 rows chunk the staged x differently
    w = synth.quant_weights(t, n, k, 6, 1)
    x = synth.activations(20, k, 6, 2)
    st = be.create_stream()
    y20, _ = run(be, st, t, w, x, n, k)
    for m in (1, 3, 4, 7, 16):
        ym, _ = run(be, st, t, w, x[:m], n, k)
        assert np.array_equal(bits(ym), bits(y20[:m])), f"batch of {m}"


def test_lm_head_over_repacked_rows_and_plan_refusal(be):
    t, n, k, m = synth.Q4_0, 9000, 512, 3   # more than one 8192-row argmax chunk
    w = synth.quant_weights(t, n, k, 8, 1)
    x = synth.activations(m, k, 8, 2)
    st = be.create_stream()
    y, _ = run(be, st, t, w, x, n, k)
    raw = be.import_host_readonly(w.reshape(-1))
    pk = be.repack(st, t, hb.TensorRef.of(raw), n, k)
    xb = be.import_host_readonly(x)
    lb, rb, ib = be.allocate(m * n * 4), be.allocate(m * 12), be.allocate(m * 4)
    g = hb.GemvArgs(t, hb.TensorRef.of(pk), hb.TensorRef.of(xb), hb.TensorRef.of(lb), n, k, m, capi.GEMV_MMA_R)
    be.lm_head(st, hb.LmHeadArgs(g, hb.TensorRef.of(rb), 0, hb.TensorRef.of(ib)))
    logits, ids = np.empty((m, n), np.float32), np.empty(m, np.int32)
    be.download(st, hb.TensorRef.of(lb), logits)
    be.download(st, hb.TensorRef.of(ib), ids)
    st.wait()
    assert np.array_equal(bits(logits), bits(y)), "the head runs the same matmul"
    assert np.array_equal(ids, np.argmax(y, axis=1))
    with pytest.raises(hb.HaloError):   # the repacked variant belongs to a tensor, not to a shape bucket
        be.plan_set(t, n, k, 1, 4, capi.GEMV_MMA_R)
