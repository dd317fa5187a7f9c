"""The GDN gates epilogue of GemvArgs::gates (include/halo/backend/backend.h:299-313): the matmul over fused beta|alpha rows stores
sigmoid(beta) and a * softplus(alpha + dt_bias) instead of y.  The checker is the CPU backend's matmul (bitwise equal to the
exact-order kernel's y) followed by the gdn_gates formulas (backends/cpu/kernel_common.h:31-33) in float64; the device's expf /
log1pf sit a few ulp from the host's, so the comparison is to 1e-6."""
from __future__ import annotations

import numpy as np
import pytest

from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu
F32 = 0


def gates(y: np.ndarray, n_v: int, dt_bias: np.ndarray, a: np.ndarray) -> np.ndarray:
    y = y.astype(np.float64)
    out = np.empty_like(y)
    out[:, :n_v] = 1.0 / (1.0 + np.exp(-y[:, :n_v]))
    t = y[:, n_v:] + dt_bias.astype(np.float64)
    out[:, n_v:] = a.astype(np.float64) * np.where(t > 20.0, t, np.log1p(np.exp(np.minimum(t, 20.0))))
    return out


def run(be, st, t, w, x, rows, cols, n_v, dt_bias, a, variant):
    n_vec = x.shape[0]
    wb = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
    xb = be.import_host_readonly(np.ascontiguousarray(x, np.float32))
    db = be.import_host_readonly(np.ascontiguousarray(dt_bias, np.float32))
    ab = be.import_host_readonly(np.ascontiguousarray(a, np.float32))
    yb = be.allocate(n_vec * rows * 4)
    args = hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), rows, cols, n_vec, variant, gates_n_v=n_v,
                       gates_dt_bias=hb.TensorRef.of(db), gates_a=hb.TensorRef.of(ab))
    be.gemv(st, args)
    y = np.empty((n_vec, rows), np.float32)
    be.download(st, hb.TensorRef.of(yb), y)
    st.wait()
    return y


@pytest.mark.parametrize("t", [synth.Q8_0, F32])
@pytest.mark.parametrize("variant", [0, capi.GEMV_EXACT8, capi.GEMV_WARP_F32])
@pytest.mark.parametrize("n_vec", [1, 5])
def test_gates_epilogue_matches_matmul_then_gdn_gates(checker, t, variant, n_vec):
    if t == F32 and variant == capi.GEMV_WARP_F32:
        pytest.skip("the fp32 streaming kernel takes block formats only")
    be = hb.CudaBackend(0)
    st = be.create_stream()
    n_v, cols = 48, 5120
    rows = 2 * n_v
    if t == F32:
        w = (synth.normal_f32(0, 5, (rows, cols)) * 0.02).astype(np.float32)
    else:
        w = synth.quant_weights(t, rows, cols, seed=4)
    x = (synth.activations(n_vec, cols, seed=5) * 0.02).astype(np.float32)  # y of a few units: both gate functions away from saturation
    rng = np.random.default_rng(6)
    dt_bias = rng.uniform(-2, 2, n_v).astype(np.float32)
    a = (-np.exp(rng.uniform(-3, 1, n_v))).astype(np.float32)
    want = gates(checker.gemv(t, w, x, rows, cols), n_v, dt_bias, a)
    got = run(be, st, t, w, x, rows, cols, n_v, dt_bias, a, variant)
    tol = 1e-6 if variant == capi.GEMV_EXACT8 or t == F32 else 1e-4   # the streaming kernel's y differs from the CPU's in the last bits
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) <= tol
    assert np.all((got[:, :n_v] >= 0) & (got[:, :n_v] <= 1)) and np.all(got[:, n_v:] <= 0)
    assert 0.05 < np.mean(got[:, :n_v]) < 0.95


def test_softplus_large_argument_branch():
    """alpha + dt_bias above 20 takes the identity branch, like cpu::softplus."""
    be = hb.CudaBackend(0)
    st = be.create_stream()
    n_v, cols = 2, 32
    w = np.zeros((4, cols), np.float32)
    w[2, 0], w[3, 0] = 25.0, 19.0
    x = np.zeros((1, cols), np.float32)
    x[0, 0] = 1.0
    got = run(be, st, F32, w, x, 4, cols, n_v, np.zeros(n_v, np.float32), np.array([2.0, 2.0], np.float32), capi.GEMV_EXACT8)
    assert got[0, 0] == 0.5 and got[0, 1] == 0.5
    assert got[0, 2] == 50.0 and abs(got[0, 3] - 2.0 * np.log1p(np.exp(19.0))) <= 1e-5


def test_gates_refusals():
    be = hb.CudaBackend(0)
    st = be.create_stream()
    cols = 512
    ones = be.import_host_readonly(np.ones(64, np.float32))

    def code(t, rows, n_v, variant=0, **kw):
        w = synth.quant_weights(t, rows, cols, seed=1)
        wb = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
        xb = be.import_host_readonly(synth.activations(1, cols, seed=2))
        yb = be.allocate(rows * 4)
        a = hb.GemvArgs(t, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), rows, cols, 1, variant, gates_n_v=n_v,
                        gates_dt_bias=hb.TensorRef.of(ones), gates_a=hb.TensorRef.of(ones), **kw)
        try:
            be.gemv(st, a)
        except hb.HaloError as e:
            return e.code
        return None

    assert code(synth.Q8_0, 32, 16) is None
    assert code(synth.Q8_0, 32, 15) == "Kernel"                       # rows != 2 * n_v
    assert code(synth.Q4_K, 32, 16) == "Unsupported"                  # F32 / Q8_0 weights only
    assert code(synth.Q8_0, 32, 16, norm_w=hb.TensorRef.of(ones)) == "Unsupported"
    assert code(synth.Q8_0, 32, 16, capi.GEMV_MMA_R) == "Unsupported"  # a kernel without the epilogue
    assert code(synth.Q8_0, 200, 100) == "Kernel"                     # dt_bias / a views shorter than n_v
