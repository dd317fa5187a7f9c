"""Tune the real kernels on the GPU, persist, reopen, look up, install the plan, and run through it."""
from __future__ import annotations

import numpy as np
import pytest

from halo_b200 import backend as hb
from halo_b200 import capi, synth
from halo_b200.autotune import ProfileDb, TuneOptions, b200_profile_key, select_kernel, tune
from halo_b200.autotune import tuner as T
from halo_b200.autotune.cuda_ops import CudaGemvTunable
from halo_b200.autotune.key import T_BUCKETS

pytestmark = pytest.mark.gpu


def test_tune_persist_lookup_and_plan(tmp_path):
    be = hb.CudaBackend(0)
    key = b200_profile_key(be.info(), "synthetic: q4_k 4096x2048 seed 0")
    assert key.gpu_arch == "sm_100a" and key.isa_target == "sm_100a" and key.rocm_version == "" and key.vulkan_version == ""
    rows, cols = 4096, 2048
    db = ProfileDb(tmp_path / "profile.db")
    db.record_tier_bandwidth(key, tier="vram", processor="gpu", label="hbm3e copy (measured)", threads=0, buffer_bytes=1 << 31,
                             read_gbps=6545.9, write_gbps=6545.9, copy_gbps=6545.9)
    results = {}
    opts = TuneOptions()  # the reference's acceptance: cv <= 5 %; a timed sample is 96 launches long, not one
    for bucket, lo, hi in T_BUCKETS[:2]:
        op = CudaGemvTunable(be, synth.Q4_K, rows, cols, hi, bucket, copies=8, launches_per_run=96)
        names = {c.get("variant") for c in op.candidates()}
        assert {capi.GEMV_EXACT8, capi.GEMV_WARP_F32, capi.GEMV_MMA_F16X2, capi.GEMV_MMA_I8X2} <= names and capi.GEMM_TCGEN05_F16 not in names
        for _attempt in range(3):  # a neighbour on a shared host can make one run noisy: tune again rather than loosen the 5 %
            results[bucket] = tune(db, key, [op], opts)[0]
            if all(c.stability == "stable" for c in results[bucket].candidates if c.measured):
                break
        assert results[bucket].winner is not None
        assert all(c.valid for c in results[bucket].candidates), "every registered decode variant must pass validation on Q4_K"
        # the bit-exact variant is never the fastest: a tuner that picked it would point at a timing bug
        assert results[bucket].winner.get("variant") != capi.GEMV_EXACT8
    db.close()
    # a fresh read-only snapshot, as the engine opens it at creation
    ro = ProfileDb(tmp_path / "profile.db", readonly=True)
    op1 = CudaGemvTunable(be, synth.Q4_K, rows, cols, 1, "1", copies=1)
    cand, source = select_kernel(ro, key, op1.key, "cuda", op1.candidates())
    assert source == "exact" and cand == results["1"].winner
    plan = T.decode_family_plan(results, op1.family)
    fams = {op1.family[c.get("variant")] for c in plan.values()}
    assert len(fams) == 1, "decode buckets must come from one numerics family"
    for (bucket, lo, hi) in T_BUCKETS[:2]:
        be.plan_set(synth.Q4_K, rows, cols, lo, hi, plan[bucket].get("variant"))
    wb = be.allocate(rows * synth.row_bytes(synth.Q4_K, cols))
    xb = be.allocate(3 * cols * 4)
    yb = be.allocate(3 * rows * 4)
    a = hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wb), hb.TensorRef.of(xb), hb.TensorRef.of(yb), rows, cols, 3)
    assert be.resolve_variant(a) == plan["2-4"].get("variant")
    a.n_vec = 1
    assert be.resolve_variant(a) == plan["1"].get("variant")
    be.plan_clear()
    assert be.resolve_variant(a) == capi.GEMV_MMA_I8X2
