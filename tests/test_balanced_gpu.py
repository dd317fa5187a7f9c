"""Corner cases of the balanced tensor-core skinny kernels (variants 3 and 7): every way the host plan can cut a matrix
(whole units with two K slices, an even split with row blocks shared by many CTAs, several units per CTA, an odd number
of super-blocks, fewer rows than one MMA tile, a partial last unit), resident and streamed x, one and two token tiles.
Each case is checked against the exact-order kernel within the summation bound, and its rows must not depend on the
batch size across the resident / streamed boundary."""
from __future__ import annotations

import ctypes as C

import numpy as np
import pytest

from conftest import bits
from gpu_util import Harness, summation_bound
from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hz():
    return Harness()


def plan_of(wtype, rows, cols, sms):
    p = capi.GemvPlan()
    assert capi.load().halo_cuda_gemv_plan(wtype, rows, cols, sms, C.byref(p)) == 0
    return p.slices, p.ctas


def run(hz, wtype, w, x, rows, cols):
    if wtype == synth.Q4_K:
        return hz.gemv(wtype, w, x, rows, cols, variant=capi.GEMV_MMA_F16X2)
    be, st = hz.be, hz.st
    raw = be.import_host_readonly(w.reshape(-1))
    pk = be.repack(st, wtype, hb.TensorRef.of(raw), rows, cols)
    xb = be.import_host_readonly(np.ascontiguousarray(x, np.float32))
    yb = be.allocate(x.shape[0] * rows * 4)
    be.gemv(st, hb.GemvArgs(wtype, hb.TensorRef.of(pk), hb.TensorRef.of(xb), hb.TensorRef.of(yb), rows, cols, x.shape[0], capi.GEMV_MMA_R))
    y = np.empty((x.shape[0], rows), np.float32)
    be.download(st, hb.TensorRef.of(yb), y)
    st.wait()
    return y


CASES = [
    # (type, rows, cols, rows of x, what the plan does on 148 SMs)
    (synth.Q4_K, 17408, 768, 5, "two slices, odd super-block count: slice 1 has one tile fewer"),
    (synth.Q4_K, 17400, 1280, 2, "two slices, last unit partial, last row block partial"),
    (synth.Q4_K, 2176, 5120, 4, "even split, 17 CTAs per unit"),
    (synth.Q4_K, 9, 5120, 16, "fewer rows than a tile: 20 CTAs share one row block"),
    (synth.Q4_K, 40000, 256, 3, "one column per unit, several units per CTA"),
    (synth.Q4_K, 5120, 6144, 17, "two token tiles (16 + 1)"),
    (synth.Q6_K, 1024, 5120, 1, "even split over 80 CTAs"),
    (synth.Q6_K, 300, 17408, 8, "streamed x, 68 columns per unit"),
    (synth.Q8_0, 17408, 1024, 2, "Q8_0 never takes two slices"),
    (synth.Q4_0, 18992, 5120, 16, "vocabulary shard of the head"),
]


@pytest.mark.parametrize("t,n,k,m,why", CASES)
def test_partition_corner_cases_against_exact_kernel(hz, checker, t, n, k, m, why):
    w = synth.quant_weights(t, n, k, 5, 1)
    x = synth.activations(max(m, 5), k, 5, 2)
    y = run(hz, t, w, x[:m], n, k)
    ref = hz.gemv(t, w, x[:m], n, k, variant=capi.GEMV_EXACT8)
    bound = summation_bound(checker.dequantize, t, w, x[:m], n, k, depth=2 * (k // 8 + 8))
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err <= bound), f"{why}: max err / bound {np.max(err / np.maximum(bound, 1e-30)):.3f}"
    assert np.max(err) <= 1e-3 * np.max(np.abs(ref))
    # rows do not depend on the batch size: one row (resident x), the batch asked for, and five rows
    y1 = run(hz, t, w, x[:1], n, k)
    y5 = run(hz, t, w, x[:5], n, k)
    assert np.array_equal(bits(y1[0]), bits(y[0])) and np.array_equal(bits(y1[0]), bits(y5[0])), why
    for r in range(min(m, 5)):
        assert np.array_equal(bits(y[r]), bits(y5[r])), f"{why}: row {r}"


def test_plans_of_the_cases_cover_both_modes(hz):
    sms = hz.be.info().sm_count
    modes = {plan_of(t, n, k, sms)[0] for t, n, k, _, _ in CASES}
    assert modes == {1, 2}
    assert plan_of(synth.Q4_K, 17408, 768, sms) == (2, min(sms, 136))


def test_repeated_calls_leave_the_shared_counters_clean(hz, checker):
    # the cross-CTA reduction resets its counters itself: the same shared-unit shape many times, interleaved with another shape
    t, n, k = synth.Q4_K, 2176, 5120
    w = synth.quant_weights(t, n, k, 9, 1)
    x = synth.activations(1, k, 9, 2)
    first = run(hz, t, w, x, n, k)
    w2 = synth.quant_weights(t, 640, 2560, 9, 2)
    x2 = synth.activations(3, 2560, 9, 3)
    other = run(hz, t, w2, x2, 640, 2560)
    for _ in range(6):
        assert np.array_equal(bits(run(hz, t, w, x, n, k)), bits(first))
        assert np.array_equal(bits(run(hz, t, w2, x2, 640, 2560)), bits(other))
