"""GPU parity of the prefill GEMM (tcgen05) against the oracle.

The reference tests its own fp16 GEMM against the fp64 sum of the ROUNDED operands' products with the bound
(cols + 4) * u * sum|h(W) h(x)| -- which proves both correctness and that the GEMM ran
(tests/unit/vulkan/test_vk_head.cpp:1005-1013) -- and gates it behind allow_gemm (:1093-1144).  Same here."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hz():
    from gpu_util import Harness
    return Harness()


def rounded_reference(checker, w, x, n, k, dtype):
    wf = checker.dequantize(synth.Q4_K, w, n * k).reshape(n, k)
    if dtype == "f16":
        hw, hx = wf.astype(np.float16).astype(np.float64), x.astype(np.float16).astype(np.float64)
    else:  # bf16: round to nearest even on the upper 16 bits
        def bf(a):
            u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
            u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16 << 16
            return u.astype(np.uint32).view(np.float32).astype(np.float64)
        hw, hx = bf(wf), bf(x)
    ref = hx @ hw.T
    mag = np.abs(hx) @ np.abs(hw).T
    return ref, mag


@pytest.mark.parametrize("variant,dtype", [(capi.GEMM_TCGEN05_F16, "f16"), (capi.GEMM_TCGEN05_BF16, "bf16")])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (64, 512, 1024), (300, 300, 512), (512, 1000, 5120), (1, 40, 256)])
def test_gemm_within_rounded_operand_bound(hz, checker, variant, dtype, m, n, k):
    w = synth.quant_weights(synth.Q4_K, n, k, 50 + m, 1)
    x = synth.activations(m, k, 50 + m, 2)
    y = hz.gemv(synth.Q4_K, w, x, n, k, variant=variant, allow_gemm=True, y_guard=8)
    ref, mag = rounded_reference(checker, w, x, n, k, dtype)
    bound = (k + 4) * 2.0**-24 * mag
    err = np.abs(y.astype(np.float64) - ref)
    assert np.all(err <= bound), f"max err/bound {np.max(err / np.maximum(bound, 1e-300)):.3f} at {np.unravel_index(np.argmax(err / np.maximum(bound, 1e-300)), err.shape)}"
    exact = checker.gemv(synth.Q4_K, w, x, n, k)
    rel = np.max(np.abs(y - exact)) / np.max(np.abs(exact))
    assert rel <= (1e-3 if dtype == "f16" else 1e-2), f"relative max error {rel:.2e}"
    if m * n >= 4096:
        assert not np.array_equal(bits(y), bits(exact)), "16-bit operands must leave a trace: did the GEMM run?"


def test_gemm_gate_only_allow_gemm_takes_the_gemm(hz):
    # without allow_gemm every row stays bitwise its own n_vec == 1 result, whatever the batch (backend.h:300-304)
    from halo_b200 import backend as hb
    n, k, m = 256, 1024, 128
    w = synth.quant_weights(synth.Q4_K, n, k, 61, 1)
    x = synth.activations(m, k, 61, 2)
    y_plain = hz.gemv(synth.Q4_K, w, x, n, k)                    # default variant, allow_gemm off
    y_gemm = hz.gemv(synth.Q4_K, w, x, n, k, allow_gemm=True)    # default variant, allow_gemm on
    y_row5 = hz.gemv(synth.Q4_K, w, x[5:6], n, k)
    assert np.array_equal(bits(y_plain[5]), bits(y_row5[0]))
    assert not np.array_equal(bits(y_gemm), bits(y_plain))
    be = hz.be
    wb = be.allocate(n * synth.row_bytes(synth.Q4_K, k))
    xb = be.allocate(m * k * 4)
    yb = be.allocate(m * n * 4)
    a = hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m)
    assert be.resolve_variant(a) == capi.GEMV_MMA_I8X2
    a.allow_gemm = True
    assert be.resolve_variant(a) == capi.GEMM_TCGEN05_F16
    a.n_vec = 8
    assert be.resolve_variant(a) == capi.GEMV_MMA_I8X2           # decode-sized batches never take the GEMM


def test_gemm_config2_full_size_against_the_skinny_kernel(hz):
    # the prefill shape: Q4_K 17408 x 5120, M = 512; the tensor-core skinny kernel (near-fp32 accuracy, itself checked
    # against the oracle at this shape) is the yardstick, so the CPU does not have to run 9e10 multiply-adds
    n, k, m = 17408, 5120, 512
    w = synth.quant_weights(synth.Q4_K, n, k, 0, 1)
    x = synth.activations(m, k, 0, 2)
    y = hz.gemv(synth.Q4_K, w, x, n, k, variant=capi.GEMM_TCGEN05_F16, allow_gemm=True)
    ref = hz.gemv(synth.Q4_K, w, x, n, k, variant=capi.GEMV_MMA_F16X2)
    rel = np.max(np.abs(y - ref)) / np.max(np.abs(ref))
    assert rel <= 1e-3, f"relative max error {rel:.2e}"


# ---- the same GEMM over repacked Q6_K / Q8_0 / Q4_0 rows -------------------------------------------------------------------------
def run_repacked(be, t, w, x, n, k, variant, allow_gemm=True):
    from halo_b200 import backend as hb
    st = be.create_stream()
    m = x.shape[0]
    raw = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
    pk = be.repack(st, t, hb.TensorRef.of(raw), n, k)
    xb = be.import_host_readonly(np.ascontiguousarray(x, np.float32))
    yb = be.allocate(m * n * 4)
    a = hb.GemvArgs(t, hb.TensorRef.of(pk), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m, variant, allow_gemm=allow_gemm)
    chosen = be.resolve_variant(a)
    be.gemv(st, a)
    y = np.empty((m, n), np.float32)
    be.download(st, hb.TensorRef.of(yb), y)
    st.wait()
    for b in (raw, pk, xb, yb):
        b.free()
    return y, chosen


@pytest.mark.parametrize("t", [synth.Q6_K, synth.Q8_0, synth.Q4_0])
@pytest.mark.parametrize("variant,dtype", [(capi.GEMM_TCGEN05_F16_R, "f16"), (capi.GEMM_TCGEN05_BF16_R, "bf16")])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (64, 512, 1024), (300, 300, 512), (512, 1000, 5120), (130, 700, 17408)])
def test_repacked_gemm_within_rounded_operand_bound(hz, checker, t, variant, dtype, m, n, k):
    w = synth.quant_weights(t, n, k, 70 + m, 1)
    x = synth.activations(m, k, 70 + m, 2)
    y, chosen = run_repacked(hz.be, t, w, x, n, k, variant)
    assert chosen == variant
    wf = checker.dequantize(t, w, n * k).reshape(n, k)
    if dtype == "f16":
        hw, hx = wf.astype(np.float16).astype(np.float64), x.astype(np.float16).astype(np.float64)
    else:
        def bf(a):
            u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
            u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16 << 16
            return u.astype(np.uint32).view(np.float32).astype(np.float64)
        hw, hx = bf(wf), bf(x)
    ref, mag = hx @ hw.T, np.abs(hx) @ np.abs(hw).T
    bound = (k + 4) * 2.0**-24 * mag
    err = np.abs(y.astype(np.float64) - ref)
    assert np.all(err <= bound), f"max err/bound {np.max(err / np.maximum(bound, 1e-300)):.3f} at {np.unravel_index(np.argmax(err / np.maximum(bound, 1e-300)), err.shape)}"
    exact = checker.gemv(t, w, x, n, k)
    rel = np.max(np.abs(y - exact)) / np.max(np.abs(exact))
    assert rel <= (1e-3 if dtype == "f16" else 1e-2), f"relative max error {rel:.2e}"
    assert not np.array_equal(bits(y), bits(exact)), "16-bit operands must leave a trace: did the GEMM run?"


@pytest.mark.parametrize("t", [synth.Q6_K, synth.Q8_0, synth.Q4_0])
def test_repacked_tensor_takes_the_gemm_only_with_consent_and_a_prefill_sized_batch(hz, t):
    n, k, m = 256, 1024, 128
    w = synth.quant_weights(t, n, k, 62, 1)
    x = synth.activations(m, k, 62, 2)
    decode_variant = hz.be.repacked_variant(t, k)
    y_plain, v_plain = run_repacked(hz.be, t, w, x, n, k, decode_variant, allow_gemm=False)
    y_gemm, v_gemm = run_repacked(hz.be, t, w, x, n, k, decode_variant, allow_gemm=True)
    y_row5, _ = run_repacked(hz.be, t, w, x[5:6], n, k, decode_variant, allow_gemm=False)
    y_few, v_few = run_repacked(hz.be, t, w, x[:8], n, k, decode_variant, allow_gemm=True)
    assert v_plain == decode_variant and v_gemm == capi.GEMM_TCGEN05_F16_R and v_few == decode_variant
    assert np.array_equal(bits(y_plain[5]), bits(y_row5[0])) and np.array_equal(bits(y_few), bits(y_plain[:8]))
    assert not np.array_equal(bits(y_gemm), bits(y_plain))
    assert np.max(np.abs(y_gemm - y_plain)) <= 1e-3 * np.max(np.abs(y_plain))
