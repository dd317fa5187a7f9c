"""The C restatement against the reference's own outputs (committed fixtures), against
gguf-py's dequantizer (inside the same fixtures) and against the reference's hand-built
known-answer blocks.  CPU only."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits, golden, sha256
from halo_b200 import synth

TYPES = (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K)


def test_fp16_widening_all_inputs(oracle_c):
    g = golden("fp16.npz")
    got = np.array([np.float32(oracle_c.fp16_to_fp32(h)) for h in range(65536)], np.float32).view(np.uint32)
    # NaN payloads included: the widening is a pure bit operation
    assert np.array_equal(got, g["widen_bits"])


def test_fp16_narrowing_sample_and_edges(oracle_c):
    g = golden("fp16.npz")
    src = g["narrow_src_bits"].view(np.float32)
    got = np.array([oracle_c.fp32_to_fp16(float(f)) for f in src], np.uint16)
    assert np.array_equal(got, g["narrow"])


def test_row_bytes_geometry(oracle_c):
    # the reference's own geometry pins (tests/unit/tensor/test_dequant.cpp:37-50)
    assert oracle_c.row_bytes(synth.F32, 5120) == 20480
    assert oracle_c.row_bytes(synth.Q6_K, 5120) == 20 * 210
    assert oracle_c.row_bytes(synth.Q4_0, 5120) == 160 * 18
    assert oracle_c.row_bytes(synth.Q8_0, 0) == 0
    assert oracle_c.row_bytes(synth.Q4_K, 5120) == 2880
    assert oracle_c.row_bytes(synth.Q6_K, 17408) == 14280
    assert oracle_c.row_bytes(synth.Q8_0, 17408) == 18496
    assert oracle_c.row_bytes(synth.Q4_K, 100) == -1   # not a multiple of 256: Error(Model)
    assert oracle_c.row_bytes(synth.F32, -1) == -1
    assert oracle_c.row_bytes(synth.Q8_0, (2**63 - 1) // 32 * 32) == -1  # overflow
    assert oracle_c.row_bytes(5, 32) == -8             # a removed ggml type id: Error(Unsupported)
    for t in TYPES:
        assert synth.row_bytes(t, 5120) == oracle_c.row_bytes(t, 5120)


def test_q8_0_hand_built_block(oracle_c):
    # tests/unit/tensor/test_dequant.cpp:52-59
    blk = np.zeros(34, np.uint8)
    blk[0:2] = np.array([0.5], np.float16).view(np.uint8)
    blk[2:] = (np.arange(32) - 16).astype(np.int8).view(np.uint8)
    y = oracle_c.dequantize(synth.Q8_0, blk, 32)
    assert np.array_equal(y, 0.5 * (np.arange(32, dtype=np.float32) - 16))


def test_q4_0_hand_built_block_nibble_order(oracle_c):
    # low nibbles -> elements 0..15, high nibbles -> 16..31 (tests/unit/tensor/test_dequant.cpp:61-72)
    blk = np.zeros(18, np.uint8)
    blk[0:2] = np.array([2.0], np.float16).view(np.uint8)
    j = np.arange(16)
    blk[2:] = ((15 - j) << 4 | j).astype(np.uint8)
    y = oracle_c.dequantize(synth.Q4_0, blk, 32)
    assert np.array_equal(y[:16], 2.0 * (j - 8).astype(np.float32))
    assert np.array_equal(y[16:], 2.0 * (7 - j).astype(np.float32))


def test_dequantize_rejects_partial_blocks(oracle_c):
    src = np.zeros(210, np.uint8)
    with pytest.raises(ValueError):
        oracle_c.dequantize(synth.Q6_K, src, 255)
    assert oracle_c.dequantize(synth.Q6_K, src, 0).size == 0


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("label", ["rand", "cfg"])
def test_dequant_bit_exact_vs_reference_and_gguf(oracle_c, t, label):
    g = golden("dequant.npz")
    name = synth.TYPE_NAMES[t]
    w, want = g[f"{name}_{label}_bytes"], g[f"{name}_{label}_f32"]
    got = oracle_c.dequantize(t, w, want.size)
    assert np.array_equal(bits(got), bits(want))
    # a deliberately misaligned source gives the same bits (tests/unit/tensor/test_quant_blocks.cpp:44-101)
    buf = np.zeros(w.size + 3, np.uint8)
    buf[3:] = w.reshape(-1)
    assert np.array_equal(bits(oracle_c.dequantize(t, buf[3:], want.size)), bits(want))


def test_generator_is_stable():
    # the recipe-addressed weights of the fixtures must regenerate to the same bytes
    g = golden("gemv.npz")
    for i in range(int(g["n_cases"][0])):
        t, n, k, m, seed = (int(v) for v in g[f"c{i}_meta"])
        w = synth.quant_weights(t, n, k, seed, 1)
        assert sha256(w) == g[f"c{i}_w_sha"].tobytes(), f"case {i}"


def test_gemv_bitwise_vs_reference_outputs(oracle_c):
    g = golden("gemv.npz")
    for i in range(int(g["n_cases"][0])):
        t, n, k, m, seed = (int(v) for v in g[f"c{i}_meta"])
        w = synth.quant_weights(t, n, k, seed, 1)
        y = oracle_c.gemv(t, w, g[f"c{i}_x"], n, k)
        assert np.array_equal(bits(y), bits(g[f"c{i}_y"])), f"case {i}: type {t} {n}x{k} m={m}"


def test_gemv_thread_count_invariance(oracle_c):
    # tests/unit/cpu_kernels/test_ops.cpp:517-565: results are bit-identical for any thread count
    w = synth.quant_weights(synth.Q4_K, 100, 1024, 3, 1)
    x = synth.activations(5, 1024, 3, 2)
    y1 = oracle_c.gemv(synth.Q4_K, w, x, 100, 1024, threads=1)
    for th in (2, 3, 7):
        assert np.array_equal(bits(y1), bits(oracle_c.gemv(synth.Q4_K, w, x, 100, 1024, threads=th)))


def test_gemv_batch_rows_equal_single_row_calls(oracle_c):
    # every row of a batch is bitwise its own n_vec == 1 gemv (include/halo/backend/backend.h:300-304)
    w = synth.quant_weights(synth.Q6_K, 33, 512, 4, 1)
    x = synth.activations(6, 512, 4, 2)
    y = oracle_c.gemv(synth.Q6_K, w, x, 33, 512)
    for t in range(6):
        assert np.array_equal(bits(y[t]), bits(oracle_c.gemv(synth.Q6_K, w, x[t:t + 1], 33, 512)[0]))


def test_gemv_within_fp64_bound(oracle_c):
    # Model-R tolerance 8*sqrt(n)*eps*sum|terms| (tests/unit/cpu_kernels/tolerance.h:13-17, 46-48)
    for t in TYPES:
        n, k = 24, 2048
        w = synth.quant_weights(t, n, k, 9, 1)
        x = synth.activations(2, k, 9, 2)
        y = oracle_c.gemv(t, w, x, n, k)
        wf = oracle_c.dequantize(t, w, n * k).reshape(n, k).astype(np.float64)
        ref = x.astype(np.float64) @ wf.T
        bound = 8 * np.sqrt(k) * 2.0**-24 * (np.abs(x.astype(np.float64)) @ np.abs(wf).T)
        assert np.all(np.abs(y - ref) <= bound)
        assert oracle_c.vec_dot_row(t, w[0], x[0]) == np.float32(ref[0, 0])


def test_dot_order(oracle_c):
    # 8 interleaved lanes, pairwise combine, sequential tail (backends/cpu/kernel_common.h:16-27)
    rng = np.random.default_rng(0)
    a = rng.standard_normal(77).astype(np.float32)
    b = rng.standard_normal(77).astype(np.float32)
    acc = np.zeros(8, np.float32)
    for i in range(0, 72, 8):
        acc = (acc + a[i:i + 8] * b[i:i + 8]).astype(np.float32)
    tail = np.float32(0)
    for i in range(72, 77):
        tail = np.float32(tail + np.float32(a[i] * b[i]))
    s = np.float32(np.float32(np.float32(acc[0] + acc[4]) + np.float32(acc[1] + acc[5])) +
                   np.float32(np.float32(acc[2] + acc[6]) + np.float32(acc[3] + acc[7])))
    assert oracle_c.dot(a, b) == np.float32(s + tail)


@pytest.mark.parametrize("name", ["q8_0", "q4_k"])
def test_lm_head_vs_reference_outputs(oracle_c, name):
    g = golden("lm_head.npz")
    t, V, E, n, seed = (int(v) for v in g[f"{name}_meta"])
    w = synth.quant_weights(t, V, E, seed, 1)
    assert sha256(w) == g[f"{name}_w_sha"].tobytes()
    x = g[f"{name}_x"]
    res, logits, ids = oracle_c.lm_head(t, w, x, V, E)
    assert np.array_equal(res, g[f"{name}_result"])
    assert np.array_equal(bits(logits), bits(g[f"{name}_logits"]))
    assert np.array_equal(ids, g[f"{name}_ids"])
    # the winner is the first strictly greatest logit, across the 8192-row slab boundary
    for i in range(n):
        assert int(res[i, 0]) == int(np.argmax(logits[i]))
    res_v, _, ids_v = oracle_c.lm_head(t, w, x, V, E, valid_rows=5000, want_logits=False)
    assert np.array_equal(res_v, g[f"{name}_result_valid5000"])
    assert np.array_equal(ids_v, g[f"{name}_ids_valid5000"])
    assert np.all(res_v[:, 0] < 5000)
    x2 = x.copy()
    x2[1, 0] = np.nan
    res_n, _, ids_n = oracle_c.lm_head(t, w, x2, V, E, want_logits=False)
    assert np.array_equal(res_n, g[f"{name}_result_nanrow1"])
    assert np.array_equal(ids_n, g[f"{name}_ids_nanrow1"])
    assert res_n[1, 0] == 0xFFFFFFFF and res_n[1, 2] == 1 and ids_n[1] == 0
    assert np.array_equal(res_n[[0, 2]], res[[0, 2]])  # a NaN poisons only its own row


def test_reference_library_agrees_when_present(oracle_c):
    import oracle
    if not oracle.Reference.available():
        pytest.skip("the compiled reference did not travel with this tree")
    ref = oracle.Reference()
    for t in TYPES:
        w = synth.quant_weights(t, 50, 1024, 11, 1)
        x = synth.activations(3, 1024, 11, 2)
        assert np.array_equal(bits(ref.gemv(t, w, x, 50, 1024)), bits(oracle_c.gemv(t, w, x, 50, 1024)))
    # the reference rejects an output that overlaps x (tests/unit/backend/test_cpu_backend.cpp:283)
    w = synth.quant_weights(synth.Q8_0, 64, 64, 12, 1)
    x = synth.activations(1, 64, 12, 2)
    assert ref.gemv_raw(synth.Q8_0, w, x, x, 64, 64, 1) == -4
