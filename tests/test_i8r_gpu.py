"""The int8 tensor-core skinny kernels over REPACKED Q6_K / Q8_0 / Q4_0 rows (variant gemv_mma_i8x2_r) against the oracle.

Same family as gemv_mma_i8x2 (tests/test_i8_gpu.py): x is rounded to 16-bit fixed point per 256-element super-block, the
products are exact integers up to the per-group scale, so the bound is sum |w_i| * (half a step of x_i) plus the
reordered-summation bound (tests/unit/hip/test_hip_gemv.cpp:9-15), and rows are bitwise independent of the batch size
(include/halo/backend/backend.h:300-304) whatever token tile (up to 16 rows) a call is cut into."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits
from gpu_util import rounded_operand_bound
from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu
V = capi.GEMV_MMA_I8X2_R
TYPES = (synth.Q6_K, synth.Q8_0, synth.Q4_0)
FAMILY_REL = 2e-4


@pytest.fixture(scope="module")
def be():
    return hb.CudaBackend(0)


def run(be, wtype, w, x, rows, cols, variant=V, w_pad=0, x_stride=0, y_stride=0):
    """Repack on the device, then one matmul; w_pad: extra bytes between repacked rows (a multiple of 16)."""
    st = be.create_stream()
    x = np.ascontiguousarray(x, np.float32).reshape(-1, cols)
    n_vec = x.shape[0]
    raw = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
    prb = be.repacked_row_bytes(wtype, cols)
    stride = prb + w_pad
    pk = be.allocate(max(rows * stride, 16))
    rc = be.lib.halo_cuda_repack_rows(be.ctx, wtype, raw.ptr, 0, pk.ptr, stride, rows, cols, st.handle)
    assert rc == 0, capi.last_error()
    xs = x_stride or cols * 4
    xbuf = np.zeros(n_vec * xs, np.uint8)
    for t in range(n_vec):
        xbuf[t * xs:t * xs + cols * 4] = x[t].view(np.uint8)
    xb = be.import_host_readonly(xbuf)
    ys = y_stride or rows * 4
    yb = be.allocate(n_vec * ys)
    be.gemv(st, hb.GemvArgs(wtype, hb.TensorRef(pk, 0, 0, stride if w_pad else 0), hb.TensorRef(xb, 0, 0, x_stride), hb.TensorRef(yb, 0, 0, y_stride),
                            rows, cols, n_vec, variant))
    out = np.empty(n_vec * ys // 4, np.float32)
    be.download(st, hb.TensorRef.of(yb), out)
    st.wait()
    for b in (raw, pk, xb, yb):
        b.free()
    return np.stack([out[t * ys // 4:t * ys // 4 + rows] for t in range(n_vec)])


@pytest.mark.parametrize("t,n,k,m", [(synth.Q6_K, 5120, 17408, 1), (synth.Q6_K, 5120, 17408, 4), (synth.Q6_K, 5120, 17408, 8), (synth.Q8_0, 5120, 17408, 1),
                                     (synth.Q8_0, 5120, 17408, 8), (synth.Q4_0, 17408, 5120, 16), (synth.Q4_0, 5120, 17408, 16), (synth.Q4_0, 5120, 10240, 16),
                                     (synth.Q6_K, 37, 512, 3), (synth.Q8_0, 130, 256, 21), (synth.Q4_0, 13, 5120, 17), (synth.Q4_0, 1000, 2560, 5),
                                     (synth.Q4_0, 40000, 256, 2), (synth.Q6_K, 50000, 768, 5), (synth.Q8_0, 60001, 512, 16)])
def test_i8r_within_rounded_operand_bound(be, checker, t, n, k, m):
    w = synth.quant_weights(t, n, k, 0, 1)
    x = synth.activations(m, k, 0, 2)
    y = run(be, t, w, x, n, k)
    ref = checker.gemv(t, w, x, n, k)
    bound = rounded_operand_bound(checker, t, w, x, n, k)
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err <= bound), f"max err/bound {np.max(err / np.maximum(bound, 1e-30)):.3f}"
    rel = np.max(err) / np.max(np.abs(ref))
    assert rel <= FAMILY_REL, f"relative max error {rel:.2e} exceeds the family's own {FAMILY_REL}"
    if n * m >= 1000:  # not a copy of the CPU path, and not the fp16 family under another name
        assert not np.array_equal(bits(y), bits(ref))
        assert not np.array_equal(bits(y), bits(run(be, t, w, x, n, k, variant=capi.GEMV_MMA_R)))


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("n,k,rows_of_x", [(96, 2560, 20), (48, 17408, 18), (640, 6144, 17), (2176, 5120, 33), (17408, 5120, 17)])
def test_i8r_rows_do_not_depend_on_batch_size(be, t, n, k, rows_of_x):
    w = synth.quant_weights(t, n, k, 3, 1)
    x = synth.activations(rows_of_x, k, 3, 2)
    y_all = run(be, t, w, x, n, k)
    for m in (1, 2, 3, 4, 5, 7, 8, 9, 11, 12, 13, 15, 16, 17):
        if m > rows_of_x:
            continue
        ym = run(be, t, w, x[:m], n, k)
        assert np.array_equal(bits(ym), bits(y_all[:m])), f"batch of {m}"
    for r in (0, rows_of_x - 1):
        y1 = run(be, t, w, x[r:r + 1], n, k)
        assert np.array_equal(bits(y1[0]), bits(y_all[r])), f"row {r} alone"


CASES = [
    (17408, 768, 5, "two slices (where the format has them), odd super-block count"),
    (17400, 1280, 2, "last unit partial, last row block partial"),
    (2176, 5120, 16, "even split, 17 CTAs per unit, one tile of 16 rows where they fit"),
    (9, 5120, 16, "fewer rows than a tile: 20 CTAs share one row block"),
    (40000, 256, 3, "one column per unit, several units per CTA"),
    (300, 17408, 8, "68 columns per unit: a CTA keeps only the records of its own columns"),
    (5120, 17408, 2, "ranges that wrap from one unit into the next"),
]


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("n,k,m,why", CASES)
def test_i8r_partition_corner_cases_against_exact_kernel(be, checker, t, n, k, m, why):
    w = synth.quant_weights(t, n, k, 5, 1)
    x = synth.activations(max(m, 5), k, 5, 2)
    y = run(be, t, w, x[:m], n, k)
    raw = be.import_host_readonly(w.reshape(-1))
    ref = checker.gemv(t, w, x[:m], n, k) if n * k * m <= 2e8 else None
    if ref is None:
        ref = np.stack([run_exact(be, t, raw, x[r:r + 1], n, k)[0] for r in range(m)])
    raw.free()
    bound = rounded_operand_bound(checker, t, w, x[:m], n, k)
    err = np.abs(y.astype(np.float64) - ref.astype(np.float64))
    assert np.all(err <= bound), f"{why}: max err / bound {np.max(err / np.maximum(bound, 1e-30)):.3f}"
    assert np.max(err) <= FAMILY_REL * np.max(np.abs(ref))
    y1 = run(be, t, w, x[:1], n, k)
    y5 = run(be, t, w, x[:5], n, k)
    assert np.array_equal(bits(y1[0]), bits(y[0])) and np.array_equal(bits(y1[0]), bits(y5[0])), why
    for r in range(min(m, 5)):
        assert np.array_equal(bits(y[r]), bits(y5[r])), f"{why}: row {r}"


def run_exact(be, t, raw, x, n, k):
    st = be.create_stream()
    xb = be.import_host_readonly(np.ascontiguousarray(x, np.float32))
    yb = be.allocate(x.shape[0] * n * 4)
    be.gemv(st, hb.GemvArgs(t, hb.TensorRef.of(raw), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, x.shape[0], capi.GEMV_EXACT8))
    y = np.empty((x.shape[0], n), np.float32)
    be.download(st, hb.TensorRef.of(yb), y)
    st.wait()
    xb.free(), yb.free()
    return y


def test_i8r_small_batches_stream_x_where_a_cta_keeps_many_records(be):
    """10240 x 17408 under the even split leaves a CTA nineteen columns: the records of eight rows do not fit beside the Q8_0 ring, and
    the resident form would cut the batch into tiles that each read all weights.  The batch streams x instead (one pass); its rows
    equal the single-row calls (resident form, checked against the bound above) bit for bit, and the exact kernel within the family's
    tolerance."""
    t, n, k, m = synth.Q8_0, 10240, 17408, 8
    w = synth.quant_weights(t, n, k, 9, 1)
    x = synth.activations(m, k, 9, 2)
    y = run(be, t, w, x, n, k)
    raw = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
    ref = run_exact(be, t, raw, x, n, k)
    raw.free()
    assert np.max(np.abs(y - ref)) <= FAMILY_REL * np.max(np.abs(ref))
    for r in (0, 3, 7):
        y1 = run(be, t, w, x[r:r + 1], n, k)
        assert np.array_equal(bits(y1[0]), bits(y[r])), f"row {r}"
    y5 = run(be, t, w, x[:5], n, k)
    assert np.array_equal(bits(y5), bits(y[:5]))


@pytest.mark.parametrize("n,m", [(4000, 7), (5120, 5), (3500, 8)])
def test_i8r_q8_0_batches_that_convert_x_behind_their_first_tiles(be, n, m):
    """Q8_0 x 17408 under the even split at 5 - 8 rows: a CTA has more than three rounds of sixteen (record, row) pairs to convert, does
    two in front of its first tile and the rest behind tiles, each round behind its own barrier.  Ragged on purpose: row counts whose
    last unit leaves warps without tiles (they still owe their pairs), odd batch sizes.  Every row must equal its single-row call
    (which converts everything up front) bit for bit, and the exact kernel within the family's tolerance."""
    t, k = synth.Q8_0, 17408
    w = synth.quant_weights(t, n, k, 21, 1)
    x = synth.activations(m, k, 21, 2)
    y = run(be, t, w, x, n, k)
    raw = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
    ref = run_exact(be, t, raw, x, n, k)
    raw.free()
    assert np.max(np.abs(y - ref)) <= FAMILY_REL * np.max(np.abs(ref))
    for r in range(m):
        y1 = run(be, t, w, x[r:r + 1], n, k)
        assert np.array_equal(bits(y1[0]), bits(y[r])), f"row {r}"
    assert np.array_equal(bits(run(be, t, w, x, n, k)), bits(y)), "a second call gives the same bits"


@pytest.mark.parametrize("t", TYPES)
def test_i8r_strided_operands(be, t):
    n, k, m = 77, 1024, 3
    w = synth.quant_weights(t, n, k, 8, 1)
    x = synth.activations(m, k, 8, 2)
    dense = run(be, t, w, x, n, k)
    strided = run(be, t, w, x, n, k, w_pad=48, x_stride=k * 4 + 64, y_stride=n * 4 + 12)
    assert np.array_equal(bits(strided), bits(dense))


@pytest.mark.parametrize("t", TYPES)
def test_i8r_extreme_activation_ranges(be, checker, t):
    n, k = 64, 1024
    w = synth.quant_weights(t, n, k, 7, 1)
    x = synth.activations(6, k, 7, 2)
    x[0] *= 1e-20
    x[1] *= 3e20
    x[2, 5] = np.nan
    x[3] = 0.0
    x[4, 700] = np.inf
    x[5, :256] *= 1e-12
    y = run(be, t, w, x, n, k)
    ref = checker.gemv(t, w, x[[0, 1, 5]], n, k)
    for i, r in enumerate((0, 1, 5)):
        assert np.max(np.abs(y[r] - ref[i])) <= FAMILY_REL * np.max(np.abs(ref[i]))
    assert np.all(np.isnan(y[2])) and np.all(np.isnan(y[4])) and not np.any(np.isnan(y[[0, 1, 3, 5]]))
    assert not y[3].any()


def test_i8r_registry_limits_and_head(be):
    names = {i: (name, fam) for i, name, fam in be.variants(capi.OP_GEMV)}
    assert names[V] == ("gemv_mma_i8x2_r", 6) and names[capi.GEMV_MMA_I8X2][1] == 6
    t, n, k, m = synth.Q4_0, 9000, 512, 3
    w = synth.quant_weights(t, n, k, 8, 1)
    x = synth.activations(m, k, 8, 2)
    y = run(be, t, w, x, n, k)
    st = be.create_stream()
    raw = be.import_host_readonly(w.reshape(-1))
    pk = be.repack(st, t, hb.TensorRef.of(raw), n, k)
    xb = be.import_host_readonly(x)
    lb, rb, ib = be.allocate(m * n * 4), be.allocate(m * 12), be.allocate(m * 4)
    g = hb.GemvArgs(t, hb.TensorRef.of(pk), hb.TensorRef.of(xb), hb.TensorRef.of(lb), n, k, m, V)
    be.lm_head(st, hb.LmHeadArgs(g, hb.TensorRef.of(rb), 0, hb.TensorRef.of(ib)))
    logits, ids = np.empty((m, n), np.float32), np.empty(m, np.int32)
    be.download(st, hb.TensorRef.of(lb), logits)
    be.download(st, hb.TensorRef.of(ib), ids)
    st.wait()
    assert np.array_equal(bits(logits), bits(y)), "the head runs the same matmul"
    assert np.array_equal(ids, np.argmax(y, axis=1))
    with pytest.raises(hb.HaloError):  # a repacked variant belongs to a tensor, not to a shape bucket
        be.plan_set(t, n, k, 1, 4, V)
    q4k = hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(pk), hb.TensorRef.of(xb), hb.TensorRef.of(lb), 8, 256, 1, V)
    with pytest.raises(hb.HaloError) as e:  # no repacked layout for Q4_K
        be.gemv(st, q4k)
    assert e.value.code == "Unsupported"
    g.no_scratch = True
    with pytest.raises(hb.HaloError) as e:
        be.gemv(st, g)
    assert e.value.code == "Unsupported"
