"""From a profile database to a running backend: tune the matmul shapes of a workload, then install the winners as the
backend's kernel plan (the "KernelPlan" join of docs/adr/ADR-001-backend-interface.md:454-483: selection reaches dispatch
as KernelChoice{variant_id}; here halo_cuda_plan_set).  The reference consumes its profile once, at engine creation
(src/runtime/engine.cpp:680-712): open a read-only snapshot, select_kernel per operator, remember where each choice came
from ("exact", "compatible", "default")."""
from __future__ import annotations

from dataclasses import dataclass

from .. import backend as hb
from .. import capi, synth
from .cuda_ops import CudaGemvTunable
from .db import ProfileDb
from .key import T_BUCKETS, OpKey, ProfileKey, b200_profile_key
from .tuner import OpTuneResult, TuneOptions, decode_family_plan, select_kernel, tune

# (weight type, N, K) of every decode-shaped matmul the benchmark configurations name
HEADLINE_SHAPES: tuple[tuple[int, int, int], ...] = (
    (synth.Q4_K, 17408, 5120),                                                      # FFN gate / up: the headline
    (synth.Q4_K, 10240, 5120), (synth.Q4_K, 6144, 5120), (synth.Q4_K, 5120, 6144),   # Gated-DeltaNet qkv, z, out
    (synth.Q4_K, 5120, 5120), (synth.Q4_K, 1024, 5120), (synth.Q4_K, 48, 5120),      # attention q / o, k, beta / alpha
    (synth.Q6_K, 5120, 17408), (synth.Q6_K, 1024, 5120), (synth.Q8_0, 5120, 17408),  # FFN down, attention v
    (synth.Q4_0, 17408, 5120), (synth.Q4_0, 5120, 17408), (synth.Q4_0, 5120, 10240),  # the MTP-head layer
)


@dataclass
class Choice:
    wtype: int
    rows: int
    cols: int
    bucket: str
    variant: int | None
    source: str  # exact | compatible | default


def profile_key_of(be: hb.CudaBackend, workload: str = "synthetic matmul shapes, seed 0") -> ProfileKey:
    return b200_profile_key(be.info(), workload)


def tune_shapes(be: hb.CudaBackend, db: ProfileDb, key: ProfileKey, shapes=HEADLINE_SHAPES, buckets=T_BUCKETS, options: TuneOptions | None = None,
                launches_per_run: int = 48) -> dict[tuple[int, int, int], dict[str, OpTuneResult]]:
    """Tunes every (shape, batch bucket) and stores the winners.  A timed sample is `launches_per_run` back-to-back launches over
    distinct weight copies, so that a sample lasts hundreds of microseconds and the 5 % stability bar is meaningful."""
    out = {}
    for wtype, rows, cols in shapes:
        per_bucket, fam, fams = {}, None, family_of(be)
        for bucket, _lo, hi in buckets:  # the single-row bucket first: its winner fixes the numerics family of the others
            op = CudaGemvTunable(be, wtype, rows, cols, hi, bucket, launches_per_run=launches_per_run, only_family=fam)
            per_bucket[bucket] = tune(db, key, [op], options)[0]
            op.close()
            if fam is None and per_bucket[bucket].winner is not None:
                fam = fams.get(per_bucket[bucket].winner.get("variant"))
        out[(wtype, rows, cols)] = per_bucket
    return out


def family_of(be: hb.CudaBackend) -> dict[int, int]:
    return {i: fam for i, _, fam in be.variants(capi.OP_GEMV)}


def install(be: hb.CudaBackend, db: ProfileDb, key: ProfileKey, shapes=HEADLINE_SHAPES, buckets=T_BUCKETS) -> list[Choice]:
    """Looks every (shape, bucket) up and installs what the database holds.  The decode buckets of one shape must come from one
    numerics family (include/halo/backend/backend.h:300-304): the family is the one of the T = 1 choice, and a bucket whose stored
    winner belongs to another family is left to the backend's default of that family (source "default")."""
    fams = family_of(be)
    names = [c for c in _candidates(be)]
    choices = []
    for wtype, rows, cols in shapes:
        first_family = None
        for bucket, lo, hi in buckets:
            op = OpKey.matmul(bucket, cols, rows, synth.TYPE_NAMES[wtype])
            cand, source = select_kernel(db, key, op, "cuda", names)
            variant = cand.get("variant") if cand is not None else None
            if variant is not None and variant not in capi.REPACKED_VARIANTS:  # a repacked variant travels with the tensor, never with a plan
                if first_family is None:
                    first_family = fams.get(variant)
                if fams.get(variant) == first_family:
                    be.plan_set(wtype, rows, cols, lo, hi, variant)
                    choices.append(Choice(wtype, rows, cols, bucket, variant, source))
                    continue
            choices.append(Choice(wtype, rows, cols, bucket, None, "default"))
    return choices


def _candidates(be: hb.CudaBackend):
    from .candidate import Candidate
    return [Candidate.of(variant=i) for i, _, _ in be.variants(capi.OP_GEMV)]


def plan_from_results(results: dict[str, OpTuneResult], fams: dict[int, int]):
    return decode_family_plan(results, fams)
