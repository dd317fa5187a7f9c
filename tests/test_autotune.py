"""The tuner and the profile database with fake operators on a scripted clock (the reference's method,
tests/unit/autotune/autotune_test_util.h:87-131): no sleeping, temporary SQLite files."""
from __future__ import annotations

import sqlite3

import pytest

from halo_b200.autotune import Candidate, DbError, OpKey, ProfileDb, ProfileKey, TuneOptions, select_kernel, tune
from halo_b200.autotune import tuner as T
from halo_b200.autotune.key import KEY_FIELDS, pack_id

KEY = ProfileKey(model_hash="m" * 64, pack_id=pack_id("m" * 64), gpu_device="10de:2901", gpu_arch="sm_100a",
                 driver_version="nvidia-580/cuda-rt-12090", kernel_version="6.8", os="linux", power_mode="b200-hgx|default-clocks/1000W",
                 isa_target="sm_100a")
OP = OpKey.matmul("1", 5120, 17408, "q4_k")


class FakeOp:
    """Each candidate has a scripted list of durations (cycled) and a validity flag."""

    def __init__(self, script: dict[int, tuple[list[float], bool]], backend="cuda", key=OP):
        self.script, self.backend, self.key = script, backend, key
        self.calls = {v: 0 for v in script}

    def candidates(self):
        return [Candidate.of(variant=v) for v in self.script]

    def validate(self, c):
        return self.script[c.get("variant")][1]

    def run(self, c):
        v = c.get("variant")
        d = self.script[v][0]
        self.calls[v] += 1
        return d[(self.calls[v] - 1) % len(d)]


def test_candidate_text_is_canonical():
    c = Candidate.of(variant=2, rows_per_cta=4)
    assert c.to_string() == "rows_per_cta=4;variant=2"           # sorted names (tests/unit/autotune/test_key.cpp:111-123)
    assert Candidate.parse("rows_per_cta=4;variant=2") == c
    for bad in ("variant=2;rows_per_cta=4", "variant=2;", "Variant=2", "variant=2;variant=3", "variant=1.5", "variant"):
        with pytest.raises(ValueError):
            Candidate.parse(bad)
    with pytest.raises(ValueError):
        Candidate.of(variant=1 << 63)
    assert Candidate.parse("n=-9223372036854775808").get("n") == -(1 << 63)


def test_profile_key_fields_and_power_mode():
    assert [n for n, _ in KEY_FIELDS] == ["halo_version", "model_hash", "pack_id", "gpu_device", "gpu_arch", "driver_version", "rocm_version",
                                          "vulkan_version", "kernel_version", "os", "power_mode", "isa_target"]
    assert [n for n, must in KEY_FIELDS if must] == ["model_hash", "pack_id", "gpu_device", "gpu_arch", "power_mode", "isa_target"]
    KEY.validate()
    import dataclasses
    for pm in ("nobar", "unknown|a/b", "|a/b", "host|unknown/1000W", "host|clocks/unknown", "host|clocks"):
        with pytest.raises(ValueError):
            dataclasses.replace(KEY, power_mode=pm).validate()
    assert KEY.differences(KEY) == 0
    assert KEY.differences(dataclasses.replace(KEY, driver_version="x", os="y")) == 2
    assert KEY.differences(dataclasses.replace(KEY, gpu_arch="sm_90a")) is None


def test_winner_is_smallest_median_ties_go_to_smallest_text(tmp_path):
    db = ProfileDb(tmp_path / "p.db")
    op = FakeOp({3: ([100.0], True), 2: ([90.0], True), 10: ([90.0], True), 1: ([500.0], True)})
    r = tune(db, KEY, [op])[0]
    assert r.winner.to_string() == "variant=10"                  # tie at 90: "variant=10" < "variant=2" as strings
    assert r.winner_median_ns == 90.0
    assert all(op.calls[v] == 25 for v in op.calls)              # 5 warm-up + 20 timed each
    assert select_kernel(db, KEY, OP, "cuda", op.candidates()) == (Candidate.of(variant=10), "exact")


def test_unstable_and_invalid_candidates_cannot_win(tmp_path):
    db = ProfileDb(tmp_path / "p.db")
    noisy = [10.0, 30.0] * 10                                    # best median, cv far above 0.05
    op = FakeOp({1: (noisy, True), 2: ([50.0], False), 3: ([80.0], True)})
    r = tune(db, KEY, [op])[0]
    assert r.winner == Candidate.of(variant=3)
    by = {c.candidate.get("variant"): c for c in r.candidates}
    assert by[1].stability == "unstable" and by[1].rejected and by[1].measured
    assert not by[2].valid and not by[2].measured and op.calls[2] == 0


def test_all_unstable_keeps_the_existing_winner(tmp_path):
    db = ProfileDb(tmp_path / "p.db")
    tune(db, KEY, [FakeOp({2: ([70.0], True)})])
    r = tune(db, KEY, [FakeOp({2: ([10.0, 40.0], True), 3: ([5.0, 50.0], True)})])[0]
    assert r.winner is None
    assert select_kernel(db, KEY, OP, "cuda", [Candidate.of(variant=2), Candidate.of(variant=3)])[0] == Candidate.of(variant=2)


def test_nonconformant_runs_are_refused(tmp_path):
    db = ProfileDb(tmp_path / "p.db")
    with pytest.raises(ValueError):
        tune(db, KEY, [FakeOp({1: ([1.0], True)})], TuneOptions(warmup=1, iterations=3))
    tune(db, KEY, [FakeOp({1: ([1.0], True)})], TuneOptions(warmup=1, iterations=3, allow_nonconformant=True))
    with pytest.raises(ValueError):
        tune(db, KEY, [FakeOp({1: ([1.0], True)})], TuneOptions(strategy="bayesian"))


def test_winners_are_kept_per_backend_and_upserted(tmp_path):
    db = ProfileDb(tmp_path / "p.db")
    tune(db, KEY, [FakeOp({1: ([10.0], True)}, backend="cpu")])
    tune(db, KEY, [FakeOp({2: ([20.0], True), 3: ([30.0], True)}, backend="cuda")])
    tune(db, KEY, [FakeOp({2: ([20.0], True), 3: ([15.0], True)}, backend="cuda")])   # re-tune: 3 takes over
    cands = [Candidate.of(variant=v) for v in (1, 2, 3)]
    assert select_kernel(db, KEY, OP, "cpu", cands)[0] == Candidate.of(variant=1)
    assert select_kernel(db, KEY, OP, "cuda", cands)[0] == Candidate.of(variant=3)
    assert db.counts()["winning_configuration"] == 2 and db.counts()["benchmark_run"] == 5
    # a stored winner the backend no longer offers is skipped
    assert select_kernel(db, KEY, OP, "cuda", [Candidate.of(variant=2)]) == (None, "default")


def test_lookup_exact_beats_compatible_then_fewest_differences(tmp_path):
    import dataclasses
    db = ProfileDb(tmp_path / "p.db")
    k_old = dataclasses.replace(KEY, driver_version="nvidia-570/cuda-rt-12080", os="linux-old")
    k_near = dataclasses.replace(KEY, driver_version="nvidia-575/cuda-rt-12090")
    k_other_gpu = dataclasses.replace(KEY, gpu_arch="sm_90a", isa_target="sm_90a")
    tune(db, k_old, [FakeOp({1: ([10.0], True)})])
    tune(db, k_near, [FakeOp({2: ([10.0], True)})])
    tune(db, k_other_gpu, [FakeOp({3: ([10.0], True)})])
    cands = [Candidate.of(variant=v) for v in (1, 2, 3, 4)]
    assert select_kernel(db, KEY, OP, "cuda", cands) == (Candidate.of(variant=2), "compatible")   # 1 differing field beats 2
    tune(db, KEY, [FakeOp({4: ([10.0], True)})])
    assert select_kernel(db, KEY, OP, "cuda", cands) == (Candidate.of(variant=4), "exact")
    assert select_kernel(db, k_other_gpu, OP, "cuda", cands)[0] == Candidate.of(variant=3)        # must-match fields isolate GPUs


def test_database_file_format_and_refusals(tmp_path):
    p = tmp_path / "p.db"
    db = ProfileDb(p)
    tune(db, KEY, [FakeOp({2: ([20.0], True)})])
    db.record_tier_bandwidth(KEY, tier="vram", processor="gpu", label="hbm3e copy", threads=0, buffer_bytes=1 << 31, read_gbps=6545.9,
                             write_gbps=6545.9, copy_gbps=6545.9)
    db.close()
    raw = sqlite3.connect(p)                                       # plain sqlite3 reads what HALO's schema names
    assert raw.execute("PRAGMA application_id").fetchone()[0] == 0x48414C4F
    assert raw.execute("SELECT app, version FROM schema_version").fetchone() == ("halo.profile", 1)
    tables = {r[0] for r in raw.execute("SELECT name FROM sqlite_master WHERE type='table'")}
    assert tables >= {"schema_version", "hardware_profile", "tier_bandwidth", "model_profile", "operator_profile", "kernel_candidate",
                      "benchmark_run", "winning_configuration"}
    row = raw.execute("SELECT o.family, o.shape, k.backend, k.params, w.metric, w.value FROM winning_configuration w "
                      "JOIN operator_profile o ON o.id = w.operator_profile_id JOIN kernel_candidate k ON k.id = w.kernel_candidate_id").fetchone()
    assert row == ("MATMUL", "T=1,K=5120,N=17408,w=q4_k", "cuda", "variant=2", "median_ns", 20.0)
    assert raw.execute("SELECT kind, engine, mode, stability FROM benchmark_run").fetchone() == ("tune", "halo", "MATMUL/T=1,K=5120,N=17408,w=q4_k", "stable")
    ts = raw.execute("SELECT created_at FROM winning_configuration").fetchone()[0]
    assert len(ts) == 20 and ts[10] == "T" and ts.endswith("Z")
    raw.close()
    # reopen read-only: lookups work, writes are refused
    ro = ProfileDb(p, readonly=True)
    assert select_kernel(ro, KEY, OP, "cuda", [Candidate.of(variant=2)])[1] == "exact"
    with pytest.raises(DbError):
        ro.persist_tune(KEY, T.tune_one(FakeOp({2: ([1.0], True)}), TuneOptions()))
    ro.close()
    # a foreign SQLite file, a newer schema, a symlink and garbage are refused with typed errors
    foreign = tmp_path / "foreign.db"
    c = sqlite3.connect(foreign)
    c.execute("CREATE TABLE t(x)")
    c.commit()
    c.close()
    with pytest.raises(DbError) as e:
        ProfileDb(foreign)
    assert e.value.kind == "NotHaloDb"
    newer = tmp_path / "newer.db"
    ProfileDb(newer).close()
    c = sqlite3.connect(newer)
    c.execute("UPDATE schema_version SET version = 2")
    c.commit()
    c.close()
    with pytest.raises(DbError) as e:
        ProfileDb(newer)
    assert e.value.kind == "ForeignVersion"
    link = tmp_path / "link.db"
    link.symlink_to(p)
    with pytest.raises(DbError):
        ProfileDb(link)
    junk = tmp_path / "junk.db"
    junk.write_bytes(b"this is not a database" * 100)
    with pytest.raises(DbError) as e:
        ProfileDb(junk)
    assert e.value.kind in ("Corrupt", "NotHaloDb")
    with pytest.raises(DbError):
        ProfileDb(tmp_path / "absent.db", readonly=True)


def test_decode_buckets_share_one_numerics_family():
    fam = {1: 0, 2: 1, 3: 2, 6: 3}
    def res(bucket, script):
        return T.tune_one(FakeOp(script, key=OpKey.matmul(bucket, 5120, 17408, "q4_k")), TuneOptions())
    results = {"1": res("1", {2: ([40.0], True), 3: ([14.0], True), 6: ([15.0], True)}),
               "2-4": res("2-4", {2: ([30.0], True), 3: ([20.0], True), 6: ([16.0], True)})}
    plan = T.decode_family_plan(results, fam)
    # T = 1 picks family 2 (variant 3); the 2-4 bucket must stay in that family although variant 6 measured faster
    assert plan == {"1": Candidate.of(variant=3), "2-4": Candidate.of(variant=3)}


# ---- strategies and the cost model (tests/unit/autotune/test_tuner.cpp:50-118, 206-225, 391-440) -----------------------------

def _grid(a, b):
    return [Candidate.of(chunk=x, threads=y) for x in a for y in b]


def _texts(cs):
    return [c.to_string() for c in cs]


def test_strategies_exhaustive_and_grid():
    from halo_b200.autotune import plan_candidates
    every = _grid((16, 32, 64, 128), (1, 2, 4, 8))
    assert plan_candidates(every, TuneOptions(strategy="exhaustive")) == every
    g = plan_candidates(every, TuneOptions(strategy="grid", grid_stride=2))  # per dimension keep indices 0, 2 and the last
    assert _texts(g) == ["chunk=16;threads=1", "chunk=16;threads=4", "chunk=16;threads=8", "chunk=64;threads=1", "chunk=64;threads=4",
                         "chunk=64;threads=8", "chunk=128;threads=1", "chunk=128;threads=4", "chunk=128;threads=8"]
    assert plan_candidates(every, TuneOptions(strategy="grid", grid_stride=1)) == every
    with pytest.raises(ValueError):
        plan_candidates(every, TuneOptions(strategy="grid", grid_stride=0))


def test_random_strategy_is_seeded_and_pinned():
    from halo_b200.autotune import plan_candidates
    every = _grid((16, 32, 64, 128), (1, 2, 4, 8))
    o = TuneOptions(strategy="random", random_budget=5, seed=42)
    a = plan_candidates(every, o)
    assert plan_candidates(every, o) == a and len(a) == 5 and len(set(_texts(a))) == 5  # same seed, same picks, no replacement
    # the reference pins these five for seed 42 (SplitMix64 partial Fisher-Yates; tests/unit/autotune/test_tuner.cpp:82-84)
    assert _texts(a) == ["chunk=64;threads=8", "chunk=16;threads=8", "chunk=32;threads=2", "chunk=32;threads=8", "chunk=32;threads=1"]
    assert plan_candidates(every, TuneOptions(strategy="random", random_budget=5, seed=43)) != a
    assert len(plan_candidates(every, TuneOptions(strategy="random", random_budget=100, seed=42))) == len(every)
    with pytest.raises(ValueError):
        plan_candidates(every, TuneOptions(strategy="random", random_budget=0))


class CostedOp(FakeOp):
    """FakeOp whose candidates also report what they cost: `predicted` ns as bytes over a 1 GB/s tier."""

    def __init__(self, script, predicted, **kw):
        super().__init__(script, **kw)
        self.predicted = predicted

    def cost(self, c):
        from halo_b200.autotune import CostInputs
        return CostInputs(flops=0.0, bytes=int(self.predicted[c.get("variant")]), tier="vram", parallelism=1, launches=0)


def _unit_model():
    from halo_b200.autotune import CostModel
    return CostModel(bandwidth_gbps={"vram": 1.0}, bandwidth_threads=1, gflops_per_thread=1.0)


def test_heuristic_keeps_the_best_predicted_and_bayesian_is_refused(tmp_path):
    from halo_b200.autotune import UnsupportedError, plan_candidates
    op = CostedOp({v: ([100.0], True) for v in (1, 2, 3, 4, 5)}, {1: 500, 2: 100, 3: 300, 4: 100, 5: 900})
    o = TuneOptions(strategy="heuristic", heuristic_keep=3, cost_model=_unit_model())
    assert _texts(plan_candidates(op.candidates(), o, op.cost)) == ["variant=2", "variant=4", "variant=3"]  # ties: smallest text first
    with pytest.raises(ValueError):
        plan_candidates(op.candidates(), TuneOptions(strategy="heuristic", heuristic_keep=3), op.cost)  # no cost model
    with pytest.raises(ValueError):
        plan_candidates(op.candidates(), o, None)                                                       # no cost inputs
    db = ProfileDb(tmp_path / "p.db")
    with pytest.raises(UnsupportedError):
        tune(db, KEY, [op], TuneOptions(strategy="bayesian"))
    assert sum(op.calls.values()) == 0  # refused up front: nothing ran, nothing was stored
    with pytest.raises(UnsupportedError):
        tune(db, KEY, [FakeOp({})], TuneOptions(strategy="bayesian"))
    assert select_kernel(db, KEY, OP, "cuda", op.candidates()) == (None, "default")


def test_heuristic_measures_only_the_prefilter(tmp_path):
    # prediction and reality disagree: the prefilter keeps 1 and 2; 3 (really the fastest) is never measured -- the documented trade-off
    op = CostedOp({1: ([900.0], True), 2: ([800.0], True), 3: ([100.0], True)}, {1: 10, 2: 20, 3: 30})
    db = ProfileDb(tmp_path / "p.db")
    r = tune(db, KEY, [op], TuneOptions(strategy="heuristic", heuristic_keep=2, cost_model=_unit_model()))[0]
    assert len(r.candidates) == 2 and r.winner == Candidate.of(variant=2) and op.calls[3] == 0
    assert r.candidates[0].predicted is not None and r.candidates[0].predicted.total_ns == 10.0


def test_cost_model_formula_and_calibration():
    from halo_b200.autotune import CostInputs, CostModel, calibrate_gflops_per_thread
    m = CostModel(bandwidth_gbps={"host": 50.0}, bandwidth_threads=4, gflops_per_thread=2.0, launch_ns=100, sync_ns=10)
    c = CostInputs(flops=8000, bytes=50000, tier="host", parallelism=2, launches=1, syncs=3)
    e = m.estimate(c)  # compute 8000 / (2 * 2); memory 50000 / (50 * 2/4): bandwidth scales with 2 of 4 threads
    assert (e.t_compute_ns, e.t_memory_ns, e.total_ns, e.memory_bound) == (2000.0, 2000.0, 2000.0 + 30.0 + 100.0, True)
    c.parallelism = 8  # memory saturates at 4 threads, compute keeps scaling
    e = m.estimate(c)
    assert (e.t_compute_ns, e.t_memory_ns) == (500.0, 1000.0)
    c.tier = "vram"
    with pytest.raises(ValueError):
        m.estimate(c)
    c.tier, m.gflops_per_thread = "host", 0.0
    with pytest.raises(ValueError):
        m.estimate(c)
    assert calibrate_gflops_per_thread(4e6, 1e6, 2) == 2.0
    with pytest.raises(ValueError):
        calibrate_gflops_per_thread(1, 0, 1)
    rows = [{"tier": "host", "threads": 8, "read_gbps": 60.0}, {"tier": "vram", "threads": 8, "read_gbps": 200.0}]
    m = CostModel.from_measurements(rows, 1.5)
    assert m.bandwidth_gbps == {"host": 60.0, "vram": 200.0} and m.bandwidth_threads == 8
    with pytest.raises(ValueError):
        CostModel.from_measurements([rows[0], dict(rows[1], threads=4)], 1.0)
    with pytest.raises(ValueError):
        CostModel.from_measurements([dict(rows[0], read_gbps=0.0)], 1.0)
    with pytest.raises(ValueError):
        CostModel.from_measurements([], 1.0)
