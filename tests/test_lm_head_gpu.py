"""GPU parity of the fused LM head against the reference's outputs (tests/unit/backend/test_cpu_backend.cpp:479-603)."""
from __future__ import annotations

import numpy as np
import pytest

from conftest import bits, golden
from halo_b200 import backend as hb
from halo_b200 import capi, synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def hz():
    from gpu_util import Harness
    return Harness()


@pytest.mark.parametrize("name", ["q8_0", "q4_k"])
def test_lm_head_exact_variant_equals_reference_words(hz, name):
    g = golden("lm_head.npz")
    t, V, E, n, seed = (int(v) for v in g[f"{name}_meta"])
    w = synth.quant_weights(t, V, E, seed, 1)
    x = g[f"{name}_x"]
    res, logits, ids = hz.lm_head(t, w, x, V, E, variant=capi.GEMV_EXACT8)
    assert np.array_equal(res, g[f"{name}_result"])
    assert np.array_equal(bits(logits), bits(g[f"{name}_logits"]))
    assert np.array_equal(ids, g[f"{name}_ids"])
    # argmax only (no logits operand) gives the same words
    res2, _, _ = hz.lm_head(t, w, x, V, E, variant=capi.GEMV_EXACT8, want_logits=False, want_ids=False)
    assert np.array_equal(res2, res)
    res_v, _, ids_v = hz.lm_head(t, w, x, V, E, variant=capi.GEMV_EXACT8, valid_rows=5000, want_logits=False)
    assert np.array_equal(res_v, g[f"{name}_result_valid5000"])
    assert np.array_equal(ids_v, g[f"{name}_ids_valid5000"])
    x2 = x.copy()
    x2[1, 0] = np.nan
    res_n, _, ids_n = hz.lm_head(t, w, x2, V, E, variant=capi.GEMV_EXACT8, want_logits=False)
    assert np.array_equal(res_n, g[f"{name}_result_nanrow1"])
    assert np.array_equal(ids_n, g[f"{name}_ids_nanrow1"])
    dec = hb.decode_argmax(res_n)
    assert dec[1][0] == -1 and np.isnan(dec[1][1]) and dec[0][0] == int(res[0, 0])


def test_lm_head_fast_variant_index_matches_when_gap_exceeds_bound(hz, checker):
    # the argmax index must equal the CPU's whenever the CPU's top-2 gap exceeds twice the error bound
    # (tests/unit/backend/test_hip_backend.cpp:603-653)
    from gpu_util import summation_bound
    t, V, E, n = synth.Q4_0, 20000, 1024, 16
    w = synth.quant_weights(t, V, E, 77, 1)
    x = synth.activations(n, E, 77, 2)
    ref_res, ref_logits, _ = checker.lm_head(t, w, x, V, E)
    res, logits, ids = hz.lm_head(t, w, x, V, E)
    bound = summation_bound(checker.dequantize, t, w, x, V, E, depth=2 * (E // 8 + 8))
    assert np.all(np.abs(logits.astype(np.float64) - ref_logits) <= bound)
    checked = 0
    for i in range(n):
        top2 = np.sort(ref_logits[i])[-2:]
        # the winner is always the argmax of the values this backend itself produced
        assert int(res[i, 0]) == int(np.argmax(logits[i])) and ids[i] == int(res[i, 0])
        assert res[i, 1] == bits(logits[i])[int(res[i, 0])]
        if top2[1] - top2[0] > 2 * bound[i].max():
            assert int(res[i, 0]) == int(ref_res[i, 0])
            checked += 1
    assert checked >= n // 2


def test_lm_head_shard_offsets_merge_to_the_full_answer(hz, checker):
    # a vocabulary split over shards: per-shard winners carry their row offset; merging by (value desc, index asc)
    # gives the single-call answer because that order is total (backends/cpu/matmul.cpp:19-22)
    t, V, E, n = synth.Q8_0, 4096, 512, 4
    w = synth.quant_weights(t, V, E, 78, 1)
    x = synth.activations(n, E, 78, 2)
    full, _, _ = hz.lm_head(t, w, x, V, E, variant=capi.GEMV_EXACT8, want_logits=False)
    parts = [hz.lm_head(t, w[o:o + 1024], x, 1024, E, variant=capi.GEMV_EXACT8, want_logits=False, row_offset=o)[0] for o in range(0, V, 1024)]
    for i in range(n):
        cand = [(-(p[i, 1:2].view(np.float32)[0]), int(p[i, 0])) for p in parts]
        best = min(cand)
        assert best[1] == int(full[i, 0])
