"""The int8 tensor-core skinny kernels (variant gemv_mma_i8x2) against the oracle, through the C ABI.

These kernels round one operand: x becomes a 16-bit fixed-point number per 256-element super-block (two signed 8-bit
digits).  They are therefore tested the way the reference tests its rounded-operand GEMM
(tests/unit/vulkan/test_vk_head.cpp:1005-1013): against the CPU backend's result with a bound derived from the rounding
-- sum |w_i| * (half a quantisation step of x_i) -- plus the reordered-summation bound of the other fast variants
(tests/unit/hip/test_hip_gemv.cpp:9-15), plus the contract's 1e-3 of the largest output.  Everything behind the rounding
of x is integer arithmetic, so rows must be bitwise independent of the batch size (include/halo/backend/backend.h:300-304)
across every token tiling and every way the host plan cuts the matrix."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits
from gpu_util import Harness, rounded_operand_bound
from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu
V = capi.GEMV_MMA_I8X2
FAMILY_REL = 2e-4  # what the family states for itself: the largest error over the largest output on N(0, 1) activations


@pytest.fixture(scope="module")
def hz():
    return Harness()


@pytest.mark.parametrize("n,k,m", [(17408, 5120, 1), (37, 512, 3), (5120, 17408, 4), (1000, 5120, 16), (130, 256, 21), (5120, 17408, 13),
                                   (5120, 6144, 8)])
def test_i8_within_rounded_operand_bound(hz, checker, n, k, m):
    t = synth.Q4_K
    w = synth.quant_weights(t, n, k, 0, 1)
    x = synth.activations(m, k, 0, 2)
    y = hz.gemv(t, w, x, n, k, variant=V, y_guard=8)
    ref = checker.gemv(t, w, x, n, k)
    bound = rounded_operand_bound(checker, t, w, x, n, k)
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err <= bound), f"max err/bound {np.max(err / np.maximum(bound, 1e-30)):.3f}"
    rel = np.max(err) / np.max(np.abs(ref))
    assert rel <= 1e-3, f"relative max error {rel:.2e} exceeds the contract's 1e-3"
    assert rel <= FAMILY_REL, f"relative max error {rel:.2e} exceeds the family's own {FAMILY_REL}"
    if n * m >= 1000:  # not a copy of the CPU path, and not the fp16 family under another name
        assert not np.array_equal(bits(y), bits(ref))
        assert not np.array_equal(bits(y), bits(hz.gemv(t, w, x, n, k, variant=capi.GEMV_MMA_F16X2)))


@pytest.mark.parametrize("n,k,rows_of_x", [(96, 2560, 20), (48, 17408, 18), (640, 6144, 17), (2176, 5120, 33), (17408, 5120, 17)])
def test_i8_rows_do_not_depend_on_batch_size(hz, n, k, rows_of_x):
    # token tiles of up to sixteen rows (fewer where the x records of a tile would not fit), pre-staged records for batches,
    # in-kernel conversion for one row; the last shape walks ten columns per CTA, so its batches of nine rows and up stream x
    # through the double buffer while the smaller ones keep it resident
    t = synth.Q4_K
    w = synth.quant_weights(t, n, k, 3, 1)
    x = synth.activations(rows_of_x, k, 3, 2)
    y_all = hz.gemv(t, w, x, n, k, variant=V)
    for m in (1, 2, 3, 4, 5, 7, 8, 9, 11, 12, 13, 15, 16, 17):
        if m > rows_of_x:
            continue
        ym = hz.gemv(t, w, x[:m], n, k, variant=V)
        assert np.array_equal(bits(ym), bits(y_all[:m])), f"batch of {m}"
    for r in (0, rows_of_x - 1):
        y1 = hz.gemv(t, w, x[r:r + 1], n, k, variant=V)
        assert np.array_equal(bits(y1[0]), bits(y_all[r])), f"row {r} alone"


CASES = [
    (17408, 768, 5, "two slices, odd super-block count: slice 1 has one tile fewer"),
    (17400, 1280, 2, "two slices, last unit partial, last row block partial"),
    (2176, 5120, 4, "even split, 17 CTAs per unit"),
    (9, 5120, 16, "fewer rows than a tile: 20 CTAs share one row block"),
    (40000, 256, 3, "one column per unit, several units per CTA"),
    (5120, 6144, 17, "two token tiles (16 + 1)"),
    (17408, 5120, 16, "twenty super-blocks of sixteen rows do not fit: x is streamed, one tile"),
    (300, 17408, 8, "68 columns per unit: a CTA keeps only the records of its own columns"),
    (18992, 5120, 16, "vocabulary shard of the head"),
]


@pytest.mark.parametrize("n,k,m,why", CASES)
def test_i8_partition_corner_cases_against_exact_kernel(hz, checker, n, k, m, why):
    t = synth.Q4_K
    w = synth.quant_weights(t, n, k, 5, 1)
    x = synth.activations(max(m, 5), k, 5, 2)
    y = hz.gemv(t, w, x[:m], n, k, variant=V)
    ref = hz.gemv(t, w, x[:m], n, k, variant=capi.GEMV_EXACT8)
    bound = rounded_operand_bound(checker, t, w, x[:m], n, k)
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err <= bound), f"{why}: max err / bound {np.max(err / np.maximum(bound, 1e-30)):.3f}"
    assert np.max(err) <= FAMILY_REL * np.max(np.abs(ref))
    y1 = hz.gemv(t, w, x[:1], n, k, variant=V)
    y5 = hz.gemv(t, w, x[:5], n, k, variant=V)
    assert np.array_equal(bits(y1[0]), bits(y[0])) and np.array_equal(bits(y1[0]), bits(y5[0])), why
    for r in range(min(m, 5)):
        assert np.array_equal(bits(y[r]), bits(y5[r])), f"{why}: row {r}"


def test_i8_strided_operands_and_guard_bands(hz, checker):
    t, n, k, m = synth.Q4_K, 77, 1024, 3
    w = synth.quant_weights(t, n, k, 8, 1)
    x = synth.activations(m, k, 8, 2)
    rb = synth.row_bytes(t, k)
    stride = rb + 48  # rows 16-byte aligned, not dense
    buf = np.zeros(16 + n * stride, np.uint8)
    for r in range(n):
        buf[16 + r * stride:16 + r * stride + rb] = w.reshape(n, rb)[r]
    y = hz.gemv(t, buf, x, n, k, variant=V, w_stride=stride, w_offset=16, x_stride=k * 4 + 64, y_stride=n * 4 + 12, y_guard=8)
    dense = hz.gemv(t, w, x, n, k, variant=V)
    assert np.array_equal(bits(y), bits(dense))


def test_i8_extreme_activation_ranges(hz, checker):
    # per-super-block power-of-two scaling: tiny and huge rows keep their 16 bits; a NaN or an infinity poisons its own row only
    t, n, k = synth.Q4_K, 64, 1024
    w = synth.quant_weights(t, n, k, 7, 1)
    x = synth.activations(6, k, 7, 2)
    x[0] *= 1e-20
    x[1] *= 3e20
    x[2, 5] = np.nan
    x[3] = 0.0
    x[4, 700] = np.inf
    x[5, :256] *= 1e-12  # one super-block far below the others: it keeps its own scale
    y = hz.gemv(t, w, x, n, k, variant=V)
    ref = checker.gemv(t, w, x[[0, 1, 5]], n, k)
    for i, r in enumerate((0, 1, 5)):
        assert np.max(np.abs(y[r] - ref[i])) <= FAMILY_REL * np.max(np.abs(ref[i]))
    assert np.all(np.isnan(y[2])) and np.all(np.isnan(y[4])) and not np.any(np.isnan(y[[0, 1, 3, 5]]))
    assert not y[3].any()
    only_first = np.zeros((1, k), np.float32)
    only_first[0, :256] = x[5, :256]
    y_small = hz.gemv(t, w, only_first, n, k, variant=V)
    ref_small = checker.gemv(t, w, only_first, n, k)
    assert np.max(np.abs(y_small - ref_small)) <= FAMILY_REL * np.max(np.abs(ref_small))


def test_i8_repeated_calls_leave_the_shared_counters_clean(hz):
    t, n, k = synth.Q4_K, 2176, 5120
    w = synth.quant_weights(t, n, k, 9, 1)
    x = synth.activations(1, k, 9, 2)
    first = hz.gemv(t, w, x, n, k, variant=V)
    w2 = synth.quant_weights(t, 640, 2560, 9, 2)
    x2 = synth.activations(3, 2560, 9, 3)
    other = hz.gemv(t, w2, x2, 640, 2560, variant=V)
    for _ in range(6):
        assert np.array_equal(bits(hz.gemv(t, w, x, n, k, variant=V)), bits(first))
        assert np.array_equal(bits(hz.gemv(t, w2, x2, 640, 2560, variant=V)), bits(other))


def test_i8_is_the_default_for_q4k_and_knows_its_limits(hz):
    be = hz.be
    n, k, m = 256, 1024, 4
    wb = be.allocate(n * synth.row_bytes(synth.Q4_K, k) + 64)
    xb = be.allocate(m * k * 4 + 64)
    yb = be.allocate(m * n * 4)
    a = hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m)
    assert be.resolve_variant(a) == V
    for rows_of_x in (1, 16, 200):
        a.n_vec = min(rows_of_x, m)
        assert be.resolve_variant(a) == V  # one family for every decode-sized batch
    a.no_scratch = True
    assert be.resolve_variant(a) == capi.GEMV_MMA_F16X2  # the kernels that need no context scratch belong to the fp16 family
    a.no_scratch = False
    a.x = hb.TensorRef(xb, 4, 0, 0)  # x off a 16-byte boundary: the tensor-core kernels read it as float4
    assert be.resolve_variant(a) in (capi.GEMV_WARP_F32, capi.GEMV_EXACT8)  # an fp32 kernel, whichever takes the operand
    a.variant_id = V
    with pytest.raises(hb.HaloError) as e:
        be.gemv(hz.st, a)
    assert e.value.code == "Unsupported"
    q8 = hb.GemvArgs(synth.Q8_0, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), 8, 64, 1, V)
    with pytest.raises(hb.HaloError) as e:
        be.gemv(hz.st, q8)
    assert e.value.code == "Unsupported"
    names = {i: (name, fam) for i, name, fam in be.variants(capi.OP_GEMV)}
    assert names[V] == ("gemv_mma_i8x2", 6)
