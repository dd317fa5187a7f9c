"""The fused input norm of GemvArgs::norm_w (include/halo/backend/backend.h:292-298): y = W (rms_norm(x) * norm_w) from the raw row.

The checker restates the CPU backend's rms_norm (backends/cpu/ops_basic.cpp:23-31: mean from the 8-lane dot of
backends/cpu/kernel_common.h:16-27, then (x * inv) * w, never fused) and feeds the normalised row to the matmul.  The fused kernel
sums the squares in its own order -- the latitude the reference gives its fused norm -- so the comparison is to rounding, and a
case whose squares sum exactly in any order pins the rest of the arithmetic bit for bit."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits
from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu


def cpu_rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    n = x.size
    acc = np.zeros(8, np.float32)
    sq = (x * x).astype(np.float32)
    for i in range(0, n - n % 8, 8):
        acc = (acc + sq[i:i + 8]).astype(np.float32)
    tail = np.float32(0)
    for i in range(n - n % 8, n):
        tail = np.float32(tail + sq[i])
    s = np.float32(np.float32(np.float32(acc[0] + acc[4]) + np.float32(acc[1] + acc[5])) + np.float32(np.float32(acc[2] + acc[6]) + np.float32(acc[3] + acc[7])))
    s = np.float32(s + tail)
    mean = np.float32(s / np.float32(n))
    inv = np.float32(np.float32(1.0) / np.sqrt(np.float32(mean + np.float32(eps))))
    return ((x * inv).astype(np.float32) * w).astype(np.float32)


def run(be, st, t, w, x, norm_w, rows, cols, eps, variant, fused=True):
    wb = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
    if variant in capi.REPACKED_VARIANTS:
        wb = be.repack(st, t, hb.TensorRef.of(wb), rows, cols)
    xb = be.import_host_readonly(np.ascontiguousarray(x, np.float32))
    nb = be.import_host_readonly(np.ascontiguousarray(norm_w, np.float32))
    yb = be.allocate(rows * 4)
    a = hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), rows, cols, 1, variant)
    if fused:
        a.norm_w, a.norm_eps = hb.TensorRef.of(nb), eps
    be.gemv(st, a)
    y = np.empty((1, rows), np.float32)
    be.download(st, hb.TensorRef.of(yb), y)
    st.wait()
    return y


CASES = [(synth.Q4_K, 70, 2560, 0), (synth.Q4_K, 17408, 5120, 0), (synth.Q4_K, 70, 2560, capi.GEMV_MMA_F16X2),
         (synth.Q4_K, 17408, 5120, capi.GEMV_MMA_F16X2), (synth.Q6_K, 37, 3072, capi.GEMV_MMA_R), (synth.Q6_K, 5120, 17408, capi.GEMV_MMA_R),
         (synth.Q8_0, 50, 1536, capi.GEMV_MMA_R), (synth.Q4_0, 129, 2048, capi.GEMV_MMA_R), (synth.Q6_K, 37, 3072, capi.GEMV_MMA_I8X2_R),
         (synth.Q6_K, 5120, 17408, capi.GEMV_MMA_I8X2_R), (synth.Q8_0, 50, 1536, capi.GEMV_MMA_I8X2_R), (synth.Q4_0, 129, 2048, capi.GEMV_MMA_I8X2_R)]


@pytest.mark.parametrize("t,rows,cols,variant", CASES)
def test_fused_norm_matches_rms_norm_then_matmul(checker, t, rows, cols, variant):
    be = hb.CudaBackend(0)
    st = be.create_stream()
    w = synth.quant_weights(t, rows, cols, seed=0, tensor_id=7)
    x = (synth.activations(1, cols, seed=1) * 3.0).astype(np.float32)
    norm_w = (1.0 + 0.1 * synth.activations(1, cols, seed=2)).astype(np.float32).reshape(-1)
    eps = 1e-6
    xn = cpu_rms_norm(x.reshape(-1), norm_w, eps).reshape(1, cols)
    want = checker.gemv(t, w, xn, rows, cols)
    got = run(be, st, t, w, x, norm_w, rows, cols, eps, variant)
    unfused = run(be, st, t, w, xn, norm_w, rows, cols, eps, variant, fused=False)
    scale = np.max(np.abs(want))
    # variant 0 on Q4_K is the int8 family: x becomes a 16-bit fixed-point number per super-block, and a last-bit difference in the
    # normalised row may move an element by one quantisation step
    i8 = (t == synth.Q4_K and variant == 0) or variant == capi.GEMV_MMA_I8X2_R
    assert np.max(np.abs(got - want)) <= (2e-4 if i8 else 1e-5) * scale     # against the CPU backend: rms_norm, then its own matmul
    assert np.max(np.abs(got - unfused)) <= (1e-4 if i8 else 2e-6) * scale  # against this backend's matmul over the CPU's normalised row


@pytest.mark.parametrize("variant", [0, capi.GEMV_MMA_F16X2])
def test_fused_norm_is_bitwise_when_the_squares_sum_exactly(variant):
    """x of +-2^k: every partial sum of squares is exact in any order, so inv -- and with it every element of the normalised row and
    the whole product -- must equal the unfused path bit for bit."""
    be = hb.CudaBackend(0)
    st = be.create_stream()
    t, rows, cols = synth.Q4_K, 333, 5120
    rng = np.random.default_rng(5)
    x = (np.ldexp(1.0, rng.integers(-1, 3, cols)) * rng.choice([-1.0, 1.0], cols)).astype(np.float32).reshape(1, cols)
    norm_w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    w = synth.quant_weights(t, rows, cols, seed=3)
    xn = cpu_rms_norm(x.reshape(-1), norm_w, 1e-6).reshape(1, cols)
    got = run(be, st, t, w, x, norm_w, rows, cols, 1e-6, variant)
    unfused = run(be, st, t, w, xn, norm_w, rows, cols, 1e-6, variant, fused=False)
    assert np.array_equal(bits(got), bits(unfused))


def test_fused_norm_refusals():
    """Every case the kernels do not have is refused, never computed over the raw row (backend.h:296-297)."""
    be = hb.CudaBackend(0)
    st = be.create_stream()
    rows, cols = 32, 512
    nb = be.import_host_readonly(np.ones(cols, np.float32))

    def call(t, n_vec, variant, **kw):
        w = synth.quant_weights(t, rows, cols, seed=1)
        wb = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
        xb = be.import_host_readonly(synth.activations(n_vec, cols, seed=2))
        yb = be.allocate(n_vec * rows * 4)
        a = hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), rows, cols, n_vec, variant, norm_w=hb.TensorRef.of(nb), **kw)
        try:
            be.gemv(st, a)
        except hb.HaloError as e:
            return e.code
        return None

    assert call(synth.Q4_K, 1, 0) is None
    assert call(synth.Q4_K, 2, 0) == "Unsupported"                      # one x row only
    assert call(synth.Q4_K, 1, capi.GEMV_EXACT8) == "Unsupported"       # a kernel without it
    assert call(synth.Q8_0, 1, 0) == "Unsupported"                      # raw Q8_0 runs the fp32 kernel
    assert call(synth.Q4_K, 1, 0, no_scratch=True) == "Unsupported"
    assert call(synth.Q4_K, 1, 0, norm_eps=-1.0) == "Kernel"
    short = hb.GemvArgs(synth.Q4_K, norm_w=hb.TensorRef(nb, 0, 16, 0))
    with pytest.raises(hb.HaloError):
        be._resolve(short.norm_w, cols * 4, "norm_w", "MATMUL")
    h = hb.LmHeadArgs(gemv=hb.GemvArgs(synth.Q4_K, norm_w=hb.TensorRef.of(nb)))
    with pytest.raises(hb.HaloError) as e:
        be.lm_head(st, h)
    assert e.value.code == "Unsupported"
