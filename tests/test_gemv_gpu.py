"""GPU parity: the cuda backend against the oracle on the same seeded bytes, through the C ABI.

Pattern of the reference's own GPU-adapter tests (tests/unit/backend/test_hip_backend.cpp:363-397, 497-529):
(a) the CPU-order variant is bitwise equal; (b) fast variants stay within a derived summation bound AND
differ from the CPU in at least one bit somewhere (so a bitwise test is not comparing a path with itself);
odd shapes, strides, offsets and guard bands (tests/unit/hip/test_hip_gemv.cpp:200-230)."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits, golden
from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu

TYPES = (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K)


@pytest.fixture(scope="module")
def hz():
    from gpu_util import Harness
    return Harness()


# ---- bit-exact unpacking -----------------------------------------------------------------------------------

@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("label", ["rand", "cfg"])
def test_dequant_bit_exact_vs_golden(hz, t, label):
    g = golden("dequant.npz")
    name = synth.TYPE_NAMES[t]
    w, want = g[f"{name}_{label}_bytes"], g[f"{name}_{label}_f32"]
    cols = w.shape[1] // synth.BLOCK_BYTES[t] * synth.BLOCK_ELEMS[t]
    got, status = hz.dequant(t, w, 2, cols)
    assert status == 0
    assert np.array_equal(bits(got.reshape(-1)), bits(want))


@pytest.mark.parametrize("t", TYPES)
def test_get_rows_ids_and_bad_index(hz, checker, t):
    cols = 2 * synth.BLOCK_ELEMS[t] if synth.BLOCK_ELEMS[t] == 256 else 96
    w = synth.random_blocks_finite(t, 10, cols, 31, t)
    ids = [3, 0, 9, 3]
    got, status = hz.dequant(t, w, 10, cols, ids)
    assert status == 0
    for i, r in enumerate(ids):
        assert np.array_equal(bits(got[i]), bits(checker.dequantize(t, w[r], cols)))
    _, status = hz.dequant(t, w, 10, cols, [1, 10])
    assert status == 8  # kStatusBadIndex


# ---- the CPU-order variant: bitwise -------------------------------------------------------------------------

def test_exact_variant_bitwise_vs_golden_outputs(hz):
    g = golden("gemv.npz")
    for i in range(int(g["n_cases"][0])):
        t, n, k, m, seed = (int(v) for v in g[f"c{i}_meta"])
        w = synth.quant_weights(t, n, k, seed, 1)
        y = hz.gemv(t, w, g[f"c{i}_x"], n, k, variant=capi.GEMV_EXACT8, y_guard=8)
        assert np.array_equal(bits(y), bits(g[f"c{i}_y"])), f"case {i}: type {t} {n}x{k} m={m}"


@pytest.mark.parametrize("t", TYPES)
def test_exact_variant_bitwise_odd_strides_and_offsets(hz, checker, t):
    # 13 rows x 5120, 3 vectors, odd byte offset and padded row strides (tests/unit/hip/test_hip_gemv.cpp:220-227)
    n, k, m = 13, 5120, 3
    rb = synth.row_bytes(t, k)
    w = synth.quant_weights(t, n, k, 40 + t, 1)
    stride = rb + 7
    buf = np.zeros(5 + n * stride, np.uint8)
    for r in range(n):
        buf[5 + r * stride:5 + r * stride + rb] = w[r]
    x = synth.activations(m, k, 40 + t, 2)
    y = hz.gemv(t, buf, x, n, k, variant=capi.GEMV_EXACT8, w_stride=stride, w_offset=5, x_stride=k * 4 + 64, y_stride=n * 4 + 12,
                y_guard=4)
    assert np.array_equal(bits(y), bits(checker.gemv(t, w, x, n, k)))


def test_exact_variant_bitwise_cfg0_full_size(hz, checker):
    # the headline decode shape: Q4_K 17408 x 5120 (the 27B FFN gate / up projection), M = 1, seed 0
    n, k = 17408, 5120
    w = synth.quant_weights(synth.Q4_K, n, k, 0, 1)
    x = synth.activations(1, k, 0, 2)
    y = hz.gemv(synth.Q4_K, w, x, n, k, variant=capi.GEMV_EXACT8)
    assert np.array_equal(bits(y), bits(checker.gemv(synth.Q4_K, w, x, n, k)))


@pytest.mark.parametrize("t,m", [(synth.Q6_K, 1), (synth.Q6_K, 4), (synth.Q8_0, 8)])
def test_exact_variant_bitwise_cfg1_full_size(hz, checker, t, m):
    # the FFN down projection: N = 5120, K = 17408, Q6_K and Q8_0
    n, k = 5120, 17408
    w = synth.quant_weights(t, n, k, 0, 1)
    x = synth.activations(m, k, 0, 2)
    y = hz.gemv(t, w, x, n, k, variant=capi.GEMV_EXACT8)
    assert np.array_equal(bits(y), bits(checker.gemv(t, w, x, n, k)))


def test_exact_variant_f32_weights_with_tail(hz, checker):
    n, k, m = 40, 77, 3  # 77 = 9*8 + 5: exercises the sequential tail of the dot
    w = synth.quant_weights(synth.F32, n, k, 8, 1)
    x = synth.activations(m, k, 8, 2)
    y = hz.gemv(synth.F32, w, x, n, k, variant=capi.GEMV_EXACT8)
    assert np.array_equal(bits(y), bits(checker.gemv(synth.F32, w, x, n, k)))


# ---- the fast fp32 variant: bounded, batch-invariant, and not vacuous ------------------------------------------

FAST = [capi.GEMV_WARP_F32, capi.GEMV_MMA_F16X2, capi.GEMV_MMA_M1]
MMA_TYPES = (synth.Q4_K,)


def _skip_unless_supported(variant, t):
    if variant in (capi.GEMV_MMA_F16X2, capi.GEMV_MMA_M1) and t not in MMA_TYPES:
        pytest.skip("gemv_mma_f16x2 takes Q4_K weights")


@pytest.mark.parametrize("variant", FAST)
@pytest.mark.parametrize("t,n,k,m", [(synth.Q4_K, 17408, 5120, 1), (synth.Q6_K, 5120, 17408, 4), (synth.Q8_0, 5120, 17408, 8),
                                     (synth.Q4_0, 2048, 5120, 16), (synth.Q4_K, 37, 512, 3), (synth.Q6_K, 13, 5120, 17),
                                     (synth.Q4_K, 5120, 17408, 4), (synth.Q4_K, 1000, 5120, 16), (synth.Q4_K, 130, 256, 21),
                                     (synth.Q4_K, 5120, 17408, 13)])
def test_fast_variant_within_summation_bound(hz, checker, variant, t, n, k, m):
    from gpu_util import summation_bound
    _skip_unless_supported(variant, t)
    w = synth.quant_weights(t, n, k, 0, 1)
    x = synth.activations(m, k, 0, 2)
    y = hz.gemv(t, w, x, n, k, variant=variant, y_guard=8)
    ref = checker.gemv(t, w, x, n, k)
    # CPU depth: K/8 adds + 3 combines + 1 product rounding; GPU: chunk-local sums + 5 shuffle adds, plus the
    # factored scale/min products: bounded by the same order.  2 * (K/8 + 8) roundings covers both paths.
    bound = summation_bound(checker.dequantize, t, w, x, n, k, depth=2 * (k // 8 + 8))
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err <= bound), f"max err/bound {np.max(err / np.maximum(bound, 1e-30)):.3f}"
    rel = np.max(err) / np.max(np.abs(ref))
    assert rel <= 1e-3, f"relative max error {rel:.2e} exceeds the contract's 1e-3"
    if n * m >= 1000:
        assert not np.array_equal(bits(y), bits(ref)), "a fast variant that is bitwise the CPU result is suspicious"


@pytest.mark.parametrize("variant", FAST)
@pytest.mark.parametrize("t", TYPES)
def test_fast_variant_rows_do_not_depend_on_batch_size(hz, variant, t):
    # every row of a batch is bitwise its own n_vec == 1 gemv (include/halo/backend/backend.h:300-304)
    _skip_unless_supported(variant, t)
    n, k = 96, 2560
    w = synth.quant_weights(t, n, k, 3, 1)
    x = synth.activations(16, k, 3, 2)
    y16 = hz.gemv(t, w, x, n, k, variant=variant)
    for m in (1, 2, 3, 4, 5, 8, 11):
        ym = hz.gemv(t, w, x[:m], n, k, variant=variant)
        assert np.array_equal(bits(ym), bits(y16[:m])), f"batch of {m}"


def test_mma_variant_batch_invariance_across_k_chunking(hz):
    # K = 17408 makes the shared-memory staging of x chunk differently for 1, 4 and 16 rows; the bits must not move
    n, k = 48, 17408
    w = synth.quant_weights(synth.Q4_K, n, k, 6, 1)
    x = synth.activations(20, k, 6, 2)
    y20 = hz.gemv(synth.Q4_K, w, x, n, k, variant=capi.GEMV_MMA_F16X2)
    for m in (1, 4, 7, 16):
        ym = hz.gemv(synth.Q4_K, w, x[:m], n, k, variant=capi.GEMV_MMA_F16X2)
        assert np.array_equal(bits(ym), bits(y20[:m])), f"batch of {m}"


def test_mma_variant_handles_extreme_activation_ranges(hz, checker):
    # per-row power-of-two scaling keeps tiny and huge activations inside fp16; a NaN poisons only its own row
    n, k = 64, 1024
    w = synth.quant_weights(synth.Q4_K, n, k, 7, 1)
    x = synth.activations(4, k, 7, 2)
    x[0] *= 1e-6
    x[1] *= 3e4
    x[2, 5] = np.nan
    x[3] = 0.0
    y = hz.gemv(synth.Q4_K, w, x, n, k, variant=capi.GEMV_MMA_F16X2)
    ref = checker.gemv(synth.Q4_K, w, x, n, k)
    for r in (0, 1):
        assert np.max(np.abs(y[r] - ref[r])) <= 1e-4 * np.max(np.abs(ref[r]))
    assert np.all(np.isnan(y[2])) and not np.any(np.isnan(y[[0, 1, 3]]))
    assert not y[3].any()


def test_default_variant_is_registered_and_runs(hz, checker):
    n, k = 64, 1024
    w = synth.quant_weights(synth.Q4_K, n, k, 5, 1)
    x = synth.activations(2, k, 5, 2)
    y = hz.gemv(synth.Q4_K, w, x, n, k)  # variant 0
    ref = checker.gemv(synth.Q4_K, w, x, n, k)
    assert np.max(np.abs(y - ref)) <= 1e-3 * np.max(np.abs(ref))


# ---- validation parity: same error class as the CPU backend (tests/unit/backend/test_hip_backend.cpp:655-722) ---

def _args(be, wtype=synth.Q8_0, n=8, k=64, m=2):
    rb = synth.row_bytes(wtype, k)
    wb = be.allocate(n * rb)
    xb = be.allocate(m * k * 4)
    yb = be.allocate(m * n * 4)
    return hb.GemvArgs(wtype, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m)


def _code(fn):
    with pytest.raises(hb.HaloError) as e:
        fn()
    return e.value.code


def test_validation_error_classes(hz):
    be, st = hz.be, hz.st
    a = _args(be)
    a.variant_id = 99
    assert _code(lambda: be.gemv(st, a)) == "Config"           # unknown variant
    a = _args(be)
    a.y = a.x
    assert _code(lambda: be.gemv(st, a)) == "Kernel"           # y overlaps x
    a = _args(be)
    a.cols = 100
    assert _code(lambda: be.gemv(st, a)) == "Model"            # not whole blocks
    a = _args(be)
    a.wtype = 5
    assert _code(lambda: be.gemv(st, a)) == "Unsupported"      # removed ggml type
    a = _args(be)
    a.x = a.x.shifted(2)
    assert _code(lambda: be.gemv(st, a)) == "Kernel"           # fp32 operand not 4-byte aligned / too short
    a = _args(be)
    a.w = a.w.with_stride(10)
    assert _code(lambda: be.gemv(st, a)) == "Kernel"           # stride < row bytes
    a = _args(be)
    a.y = hb.TensorRef(a.y.buffer, 0, 16, 0)
    assert _code(lambda: be.gemv(st, a)) == "Kernel"           # view too small
    a = _args(be)
    a.norm_w = a.x
    assert _code(lambda: be.gemv(st, a)) == "Unsupported"      # fused norm is Vulkan-only
    a = _args(be)
    a.gates_n_v = 4
    a.norm_w = a.x
    assert _code(lambda: be.gemv(st, a)) == "Unsupported"      # gates next to a fused norm: refused, as everywhere in the reference
    a = _args(be)
    other = hb.CudaBackend(0)
    a.x = hb.TensorRef.of(other.allocate(2 * 64 * 4))
    assert _code(lambda: be.gemv(st, a)) == "Kernel"           # buffer of another backend
    a = _args(be)
    ro = be.import_host_readonly(np.zeros(2 * 8, np.float32))
    a.y = hb.TensorRef.of(ro)
    assert _code(lambda: be.gemv(st, a)) == "Kernel"           # read-only output
    a = _args(be)
    a.n_vec = 0
    be.gemv(st, a)                                             # empty call is a no-op
    a = _args(be)
    a.rows = 0
    be.gemv(st, a)
    assert _code(lambda: be.rms_norm(st, None)) == "Unsupported"  # never a silent CPU fallback
    st.wait()


def test_rejected_call_writes_nothing(hz):
    be, st = hz.be, hz.st
    a = _args(be)
    sentinel = np.full(2 * 8, 7.5, np.float32)
    be.upload(st, a.y, sentinel)
    a.variant_id = 99
    with pytest.raises(hb.HaloError):
        be.gemv(st, a)
    out = np.zeros_like(sentinel)
    be.download(st, a.y, out)
    st.wait()
    assert np.array_equal(out, sentinel)


def test_zero_filled_allocation_and_copy(hz):
    be, st = hz.be, hz.st
    b = be.allocate(4096)
    out = np.ones(1024, np.float32)
    be.download(st, hb.TensorRef.of(b), out)
    st.wait()
    assert not out.any()  # Backend::allocate is zero-filled (include/halo/backend/backend.h:523)
    src = be.import_host_readonly(np.arange(256, dtype=np.float32))
    be.copy(st, hb.TensorRef.of(src), hb.TensorRef.of(b), 1024)
    got = np.zeros(256, np.float32)
    be.download(st, hb.TensorRef(b, 0, 1024), got)
    st.wait()
    assert np.array_equal(got, np.arange(256, dtype=np.float32))
    assert _code(lambda: be.copy(st, hb.TensorRef.of(b), hb.TensorRef(b, 512), 1024)) == "Kernel"  # overlap
