"""The tuner: measure every candidate of an operator, keep the fastest valid and stable one, persist it, look it up.

Behaviour follows the reference (src/autotune/tuner.cpp:106-188, tests/unit/autotune/test_tuner.cpp:50-423):
 * a candidate whose validate() is false cannot win and is not measured;
 * each candidate runs `warmup` untimed and `iterations` timed calls; fewer than 5 + 20 is refused unless
   allow_nonconformant (include/halo/profiling/stats.h:48-63);
 * a candidate whose coefficient of variation exceeds max_cv (0.05) is unstable and cannot win;
 * the winner is the smallest median ns among valid and stable candidates, ties go to the smallest canonical string;
 * with no eligible candidate there is no winner and an existing stored winner stays;
 * winners are stored per backend label;
 * strategies decide WHICH candidates are measured: exhaustive (all), grid (per parameter every grid_stride-th distinct value
   plus the last), random (a seeded partial Fisher-Yates over SplitMix64: portable and pinned), heuristic (the heuristic_keep
   best by the cost model's prediction; needs a cost model and cost inputs); bayesian is refused before any run.
Lookup (src/autotune/lookup.cpp:72-148): an exact key match beats a compatible one; among compatible keys the fewest
differing version-tolerant fields, then the newest; a stored winner that is not among the current candidates is skipped.
"""
from __future__ import annotations

import statistics
from dataclasses import dataclass, field
from typing import Protocol

from .candidate import Candidate
from .cost_model import CostEstimate, CostInputs, CostModel
from .db import ProfileDb
from .key import OpKey, ProfileKey

MIN_WARMUP, MIN_ITERATIONS = 5, 20


class UnsupportedError(ValueError):
    """The reference's Error(Unsupported): a documented feature this version does not have."""


class TunableOp(Protocol):
    key: OpKey
    backend: str

    def candidates(self) -> list[Candidate]: ...
    def validate(self, c: Candidate) -> bool: ...
    def run(self, c: Candidate) -> float: ...  # one call; returns its duration in ns (device time where available)
    # optional: def cost(self, c: Candidate) -> CostInputs | None  (what the candidate does, for the cost model)


@dataclass
class TuneOptions:
    warmup: int = MIN_WARMUP
    iterations: int = MIN_ITERATIONS
    max_cv: float = 0.05
    allow_nonconformant: bool = False
    strategy: str = "exhaustive"  # exhaustive | grid | random | heuristic (bayesian: refused)
    grid_stride: int = 1
    random_budget: int = 8
    seed: int = 0
    heuristic_keep: int = 4
    cost_model: CostModel | None = None


@dataclass
class CandidateResult:
    candidate: Candidate
    valid: bool = True
    measured: bool = False
    stability: str = "unknown"  # stable | unstable
    stats: dict = field(default_factory=dict)
    rejected: str | None = None
    predicted: CostEstimate | None = None

    def to_json(self) -> dict:
        return {"candidate": self.candidate.to_string(), "valid": self.valid, "measured": self.measured, "stability": self.stability,
                "stats": self.stats, "rejected": self.rejected, "predicted": self.predicted.to_json() if self.predicted else None}


@dataclass
class OpTuneResult:
    key: OpKey
    backend: str
    strategy: str
    candidates: list[CandidateResult]
    winner: Candidate | None = None
    winner_median_ns: float = 0.0


def sample_stats(samples: list[float]) -> dict:
    med = statistics.median(samples)
    mean = statistics.fmean(samples)
    sd = statistics.pstdev(samples) if len(samples) > 1 else 0.0
    return {"n": len(samples), "median": med, "mean": mean, "min": min(samples), "max": max(samples), "stddev": sd,
            "cv": sd / mean if mean > 0 else 0.0}


_M64 = (1 << 64) - 1


def _splitmix64(state: int) -> tuple[int, int]:
    state = (state + 0x9E3779B97F4A7C15) & _M64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return state, z ^ (z >> 31)


def _op_cost(op, c: Candidate):
    f = getattr(op, "cost", None)
    return f(c) if f is not None else None


def plan_candidates(all_: list[Candidate], o: TuneOptions, cost=None) -> list[Candidate]:
    """The candidates a strategy measures, in order (src/autotune/tuner.cpp:36-104)."""
    if o.strategy == "exhaustive":
        return list(all_)
    if o.strategy == "random":
        if o.random_budget < 1:
            raise ValueError("tune: random_budget must be >= 1 (Config)")
        pool, k, state = list(all_), min(o.random_budget, len(all_)), o.seed & _M64
        for i in range(k):  # j uniform-ish in [i, n): the high 64 bits of r * (n - i)
            state, r = _splitmix64(state)
            j = i + ((r * (len(pool) - i)) >> 64)
            pool[i], pool[j] = pool[j], pool[i]
        return pool[:k]
    if o.strategy == "grid":
        if o.grid_stride < 1:
            raise ValueError("tune: grid_stride must be >= 1 (Config)")
        values: dict[str, set[int]] = {}
        for c in all_:
            for name, v in c.params:
                values.setdefault(name, set()).add(v)
        kept = {name: set(sorted(vs)[::o.grid_stride]) | {max(vs)} for name, vs in values.items()}
        return [c for c in all_ if all(v in kept[name] for name, v in c.params)]
    if o.strategy == "heuristic":
        if o.cost_model is None:
            raise ValueError("tune: HEURISTIC needs a cost model (Config)")
        if o.heuristic_keep < 1:
            raise ValueError("tune: heuristic_keep must be >= 1 (Config)")
        if cost is None:
            raise ValueError("tune: HEURISTIC needs cost inputs (Config)")
        ranked = []
        for c in all_:
            inputs = cost(c)
            if inputs is None:
                raise ValueError(f"tune: candidate {c.to_string()} has no cost inputs (Config)")
            ranked.append((o.cost_model.estimate(inputs).total_ns, c.to_string(), c))
        ranked.sort(key=lambda r: (r[0], r[1]))
        return [c for _, _, c in ranked[:o.heuristic_keep]]
    if o.strategy == "bayesian":
        raise UnsupportedError("tune: BAYESIAN strategy is not implemented (Unsupported)")
    raise ValueError(f"tune: unknown strategy {o.strategy!r} (Config)")


def tune_one(op: TunableOp, options: TuneOptions) -> OpTuneResult:
    if options.strategy == "bayesian":
        raise UnsupportedError("tune: BAYESIAN strategy is not implemented (Unsupported)")
    if not options.allow_nonconformant and (options.warmup < MIN_WARMUP or options.iterations < MIN_ITERATIONS):
        raise ValueError(f"tuner: {options.warmup} warm-up + {options.iterations} timed runs is below the {MIN_WARMUP} + {MIN_ITERATIONS} the "
                         "methodology asks for; pass allow_nonconformant to override")
    results: list[CandidateResult] = []
    everything = op.candidates()
    if not everything:
        return OpTuneResult(op.key, op.backend, options.strategy, [])
    for c in plan_candidates(everything, options, lambda cand: _op_cost(op, cand)):
        cr = CandidateResult(c)
        inputs = _op_cost(op, c)
        if inputs is not None and options.cost_model is not None:
            cr.predicted = options.cost_model.estimate(inputs)
        if not op.validate(c):
            cr.valid, cr.rejected = False, "validation failed"
            results.append(cr)
            continue
        for _ in range(options.warmup):
            op.run(c)
        cr.stats = sample_stats([float(op.run(c)) for _ in range(options.iterations)])
        cr.measured = True
        cr.stability = "stable" if cr.stats["cv"] <= options.max_cv else "unstable"
        if cr.stability != "stable":
            cr.rejected = f"cv {cr.stats['cv']:.4f} > {options.max_cv}"
        results.append(cr)
    eligible = [r for r in results if r.valid and r.measured and r.stability == "stable"]
    out = OpTuneResult(op.key, op.backend, options.strategy, results)
    if eligible:
        best = min(eligible, key=lambda r: (r.stats["median"], r.candidate.to_string()))
        out.winner, out.winner_median_ns = best.candidate, best.stats["median"]
    return out


def tune(db: ProfileDb, key: ProfileKey, ops: list[TunableOp], options: TuneOptions | None = None) -> list[OpTuneResult]:
    options = options or TuneOptions()
    if options.strategy == "bayesian":  # refused up front, before any operator runs and whatever the operators offer
        raise UnsupportedError("tune: BAYESIAN strategy is not implemented (Unsupported)")
    out = []
    for op in ops:
        r = tune_one(op, options)
        db.persist_tune(key, r)
        out.append(r)
    return out


def select_kernel(db: ProfileDb, key: ProfileKey, op: OpKey, backend: str, candidates: list[Candidate]) -> tuple[Candidate | None, str]:
    """The stored winner to run for `op` under `key`, restricted to the current candidate list, and where it came from:
    "exact", "compatible" or "default" (nothing usable stored)."""
    allowed = {c.to_string() for c in candidates}
    best = None
    for stored_key, cand, _median, created in db.winners(op, backend):
        if cand.to_string() not in allowed:
            continue  # a winner the backend no longer offers
        diff = key.differences(stored_key)
        if diff is None:
            continue
        rank = (diff, _neg_time(created))
        if best is None or rank < best[0]:
            best = (rank, cand, "exact" if diff == 0 else "compatible")
    return (None, "default") if best is None else (best[1], best[2])


def _neg_time(created: str) -> tuple:
    # newer first: ISO-8601 UTC strings sort chronologically, so negate by inverting every character code
    return tuple(-ord(ch) for ch in created)


def decode_family_plan(results: dict[str, OpTuneResult], family_of: dict[int, int]) -> dict[str, Candidate]:
    """Winners for the decode / verify buckets (T = 1 ... 16) must share one numerics family, or a row's bits would depend
    on the batch size (include/halo/backend/backend.h:300-304).  The family is the one of the T = 1 winner (single-row
    decode is the common case); every other bucket takes its fastest stable candidate inside that family."""
    first = results.get("1")
    if first is None or first.winner is None:
        return {}
    fam = family_of[first.winner.get("variant")]
    plan = {}
    for bucket, res in results.items():
        elig = [r for r in res.candidates if r.valid and r.measured and r.stability == "stable" and family_of.get(r.candidate.get("variant")) == fam]
        if elig:
            plan[bucket] = min(elig, key=lambda r: (r.stats["median"], r.candidate.to_string())).candidate
    return plan
