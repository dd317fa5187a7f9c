"""The host-side partition of the balanced skinny kernels (halo_cuda_gemv_plan): every (row block, super-block) tile is
owned exactly once, ranges are contiguous and non-empty, and the CTAs that share a unit are the ones the kernel's
last-arriver reduction will count.  Pure host arithmetic: runs without a GPU."""
from __future__ import annotations

import ctypes as C
import random

import pytest

from halo_b200 import capi, synth


def plan(wtype: int, rows: int, cols: int, sms: int = 148):
    lib = capi.load()
    p = capi.GemvPlan()
    rc = lib.halo_cuda_gemv_plan(wtype, rows, cols, sms, C.byref(p))
    assert rc == 0, capi.last_error()
    return p.slices, p.ctas, p.cols_per_unit, list(p.start[: p.ctas + 1])


def check(wtype: int, rows: int, cols: int, sms: int = 148):
    ks, ctas, cpu, start = plan(wtype, rows, cols, sms)
    nb, n_rb, r_blocks = cols // 256, (rows + 15) // 16, 16 // ks
    assert ks in (1, 2) and 1 <= ctas <= min(sms, 160) and cpu == (nb + ks - 1) // ks
    assert start[0] == 0 and all(a < b for a, b in zip(start, start[1:])), "ranges must be contiguous and non-empty"
    units = (n_rb + r_blocks - 1) // r_blocks
    assert start[-1] == units * cpu, "the ranges must cover every column of every unit"
    seen = set()
    for c in range(ctas):
        for col in range(start[c], start[c + 1]):
            unit, k = divmod(col, cpu)
            for r in range(r_blocks):
                for s in range(ks):
                    rb, sb = unit * r_blocks + r, k * ks + s
                    if rb < n_rb and sb < nb:
                        assert (rb, sb) not in seen
                        seen.add((rb, sb))
    assert len(seen) == n_rb * nb, "every tile exactly once"
    # a CTA's range touches at most two units partially (its first and its last): two partial records per CTA suffice
    for c in range(ctas):
        partial = {col // cpu for col in (start[c], start[c + 1] - 1) if not (start[c] <= (col // cpu) * cpu and (col // cpu + 1) * cpu <= start[c + 1])}
        assert len(partial) <= 2
    return ks, ctas


def test_plan_of_the_benchmark_shapes():
    # config 0: whole units per CTA, two K slices, no row block shared between CTAs
    assert check(synth.Q4_K, 17408, 5120) == (2, 136)
    ks, ctas, cpu, start = plan(synth.Q4_K, 17408, 5120)
    assert all(s % cpu == 0 for s in start)
    # config 1: too few row blocks for that; an even split of the columns over all SMs
    assert check(synth.Q6_K, 5120, 17408) == (1, 148)
    assert check(synth.Q8_0, 5120, 17408) == (1, 148)
    # config 4 head and a tensor-parallel shard of it
    assert check(synth.Q4_0, 151936, 5120) == (1, 148)
    assert check(synth.Q4_0, 18992, 5120)[1] == 148
    # Q8_0 never takes two slices
    assert check(synth.Q8_0, 17408, 5120)[0] == 1


def test_plan_does_not_depend_on_anything_but_shape_and_sm_count():
    a = plan(synth.Q4_K, 4096, 4096)
    assert a == plan(synth.Q4_K, 4096, 4096)
    assert plan(synth.Q4_K, 4096, 4096, 132) != a or a[1] <= 132


@pytest.mark.parametrize("seed", range(4))
def test_plan_covers_random_shapes(seed):
    rng = random.Random(seed)
    for _ in range(60):
        wtype = rng.choice([synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q4_0])
        check(wtype, rng.randint(1, 40000), 256 * rng.randint(1, 70), rng.choice([148, 132, 8, 1, 160, 400]))


def test_plan_rejects_what_the_kernels_do_not_take():
    lib = capi.load()
    p = capi.GemvPlan()
    assert lib.halo_cuda_gemv_plan(synth.Q4_K, 16, 1000, 148, C.byref(p)) == capi.E_MODEL
    assert lib.halo_cuda_gemv_plan(0, 16, 1024, 148, C.byref(p)) == capi.E_UNSUPPORTED
    assert lib.halo_cuda_gemv_plan(synth.Q4_K, 0, 1024, 148, C.byref(p)) == capi.E_KERNEL


# ---- the int8 family's planner (halo_cuda_gemv_plan_i8): 1, 2, 4, 8 or 16 in-CTA slices ------------------------------------------
def plan_i8(wtype: int, rows: int, cols: int, sms: int = 148):
    lib = capi.load()
    p = capi.GemvPlan()
    rc = lib.halo_cuda_gemv_plan_i8(wtype, rows, cols, sms, C.byref(p))
    assert rc == 0, capi.last_error()
    return p.slices, p.ctas, p.cols_per_unit, list(p.start[: p.ctas + 1])


def check_i8(wtype: int, rows: int, cols: int, sms: int = 148):
    ks, ctas, cpu, start = plan_i8(wtype, rows, cols, sms)
    nb, n_rb, r_blocks = cols // 256, (rows + 15) // 16, 16 // ks
    assert ks in (1, 2, 4, 8, 16) and 1 <= ctas <= min(sms, 160) and cpu == (nb + ks - 1) // ks
    assert start[0] == 0 and all(a < b for a, b in zip(start, start[1:])), "ranges must be contiguous and non-empty"
    units = (n_rb + r_blocks - 1) // r_blocks
    assert start[-1] == units * cpu, "the ranges must cover every column of every unit"
    if ks > 1:  # slices come with whole units per CTA: nothing crosses CTAs
        assert all(s % cpu == 0 for s in start)
    owned = 0
    for c in range(ctas):
        for col in range(start[c], start[c + 1]):
            unit, k = divmod(col, cpu)
            rbs = min(r_blocks, n_rb - unit * r_blocks)
            sbs = sum(1 for s in range(ks) if k * ks + s < nb)
            owned += max(rbs, 0) * sbs
    assert owned == n_rb * nb, "every (row block, super-block) tile exactly once"
    return ks, ctas


def test_i8_plan_of_the_benchmark_shapes():
    assert check_i8(synth.Q4_K, 17408, 5120) == (2, 136)      # the headline: 136 whole units of 8 row blocks x 2 slices
    assert check_i8(synth.Q4_K, 5120, 5120) == (4, 80)        # attention q / o: 5 tiles per warp, no cross-CTA reduction
    assert check_i8(synth.Q4_K, 2176, 5120) == (16, 136)      # a tensor-parallel share of gate / up: one row block per CTA
    assert check_i8(synth.Q4_K, 48, 5120) == (16, 3)          # beta | alpha
    assert check_i8(synth.Q6_K, 5120, 17408) == (1, 148)      # 68 super-blocks of x do not fit for eight rows: even split
    assert check_i8(synth.Q8_0, 5120, 17408) == (1, 148)
    assert check_i8(synth.Q4_0, 151936, 5120) == (1, 148)     # the head: the even split walks fewer tiles than any whole-unit plan
    assert check_i8(synth.Q4_K, 5120, 256) == (1, 20)         # one super-block: nothing to slice
    # a vocabulary-sized N with a short K: sixteen slices walk one tile fewer than two, but end every tile with the slices' meeting
    assert check_i8(synth.Q4_K, 128256, 4096)[0] == 2
    assert check_i8(synth.Q4_K, 32768, 2048)[0] == 2


def test_i8_plan_is_a_function_of_shape_type_and_sm_count_only():
    a = plan_i8(synth.Q4_K, 4096, 4096)
    assert a == plan_i8(synth.Q4_K, 4096, 4096)
    # the type matters only through what fits in shared memory: Q8_0's 5 KB ring slots leave room for fewer records
    assert plan_i8(synth.Q8_0, 5120, 5120)[0] == 1 and plan_i8(synth.Q4_0, 5120, 5120)[0] == 4


@pytest.mark.parametrize("seed", range(4))
def test_i8_plan_covers_random_shapes(seed):
    rng = random.Random(100 + seed)
    for _ in range(80):
        wtype = rng.choice([synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q4_0])
        check_i8(wtype, rng.randint(1, 40000), 256 * rng.randint(1, 70), rng.choice([148, 132, 8, 1, 160, 400]))


def test_i8_plan_rejects_what_the_kernels_do_not_take():
    lib = capi.load()
    p = capi.GemvPlan()
    assert lib.halo_cuda_gemv_plan_i8(synth.Q4_K, 16, 1000, 148, C.byref(p)) == capi.E_MODEL
    assert lib.halo_cuda_gemv_plan_i8(0, 16, 1024, 148, C.byref(p)) == capi.E_UNSUPPORTED
    assert lib.halo_cuda_gemv_plan_i8(synth.Q4_K, 0, 1024, 148, C.byref(p)) == capi.E_KERNEL


# ---- how the int8 family cuts a call into launches (halo_cuda_gemv_tiles_i8) ------------------------------------------------------
MAX_TILE = {synth.Q4_K: 16, synth.Q4_0: 16, synth.Q8_0: 16, synth.Q6_K: 16}  # x rows of one launch, by format


def tiles_i8(wtype: int, rows: int, cols: int, n_vec: int, sms: int = 148):
    lib = capi.load()
    t = capi.GemvTiles()
    rc = lib.halo_cuda_gemv_tiles_i8(wtype, rows, cols, n_vec, sms, C.byref(t))
    assert rc == 0, capi.last_error()
    return t


def longest_range(wtype: int, rows: int, cols: int, sms: int = 148) -> int:
    _, _, _, start = plan_i8(wtype, rows, cols, sms)
    return max(b - a for a, b in zip(start, start[1:]))


def test_i8_tiles_of_the_benchmark_shapes():
    t = tiles_i8(synth.Q4_K, 17408, 5120, 1)
    assert (t.tile_rows, t.launches, t.conversions, t.streamed) == (1, 1, 0, 0)      # a single row is converted in the matmul kernel
    t = tiles_i8(synth.Q8_0, 5120, 17408, 8)
    assert (t.tile_rows, t.launches, t.conversions, t.streamed) == (8, 1, 0, 0)      # ten columns per CTA: 80 records, made in the kernel
    t = tiles_i8(synth.Q4_0, 17408, 5120, 16)
    assert (t.tile_rows, t.launches, t.conversions, t.streamed) == (16, 1, 1, 1)     # gate / up: twenty records of sixteen rows do not fit
    assert 2 <= t.stretch_cols <= 8
    t = tiles_i8(synth.Q4_0, 5120, 5120, 16)
    assert (t.tile_rows, t.launches, t.conversions, t.streamed) == (8, 2, 1, 0)      # q / o: a short walk, two resident tiles, ONE conversion
    t = tiles_i8(synth.Q4_0, 5120, 17408, 16)
    assert (t.tile_rows, t.launches, t.conversions, t.streamed) == (16, 1, 1, 0)     # down: a CTA keeps only its ten columns' records
    t = tiles_i8(synth.Q4_K, 17408, 5120, 17)
    assert (t.tile_rows, t.launches, t.conversions, t.streamed) == (12, 2, 1, 1)     # equal tiles of whole column groups: 12 + 5 rows


@pytest.mark.parametrize("wtype", sorted(MAX_TILE))
def test_i8_batches_are_one_pass_over_the_weights(wtype):
    """The cliff this guards against: a CTA that keeps many x records (a tall matrix under the even split, a long K) leaves the
    resident form room for one or two rows, and a batch of eight used to run as four to eight launches, each reading all weights.
    Such a batch streams x instead.  Over a grid of shapes: up to eight rows are ONE launch whatever the format; sixteen rows are
    one launch under one or two slices (streamed, or resident where a CTA keeps few records) and at most two otherwise; never
    more than one conversion launch."""
    for cols in (2048, 4096, 5120, 8192, 14336, 17408, 28672):
        for rows in (1024, 4096, 8192, 20480, 32768, 128256):
            if rows * cols > 1.3e9:
                continue
            slices = plan_i8(wtype, rows, cols)[0]
            for n_vec in (2, 4, 8, 16):
                t = tiles_i8(wtype, rows, cols, n_vec)
                where = f"{rows} x {cols} at {n_vec} rows: {t.launches} launches of {t.tile_rows} rows"
                assert t.conversions <= 1, where
                assert t.launches * t.tile_rows >= n_vec and (t.launches - 1) * t.tile_rows < n_vec, where
                if n_vec <= 8:
                    assert t.launches == 1, where
                else:
                    assert t.launches <= 2 and (t.launches == 1 or slices >= 4), where
