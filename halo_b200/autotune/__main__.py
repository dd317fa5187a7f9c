"""python -m halo_b200.autotune --db PATH [--shapes all|headline] [--strategy exhaustive|grid|random|heuristic] [--device N]

The tune driver of the cuda backend (the reference's is `halo tune`, tools/halo/tune.cpp:262-355, which wires CPU operators
only): builds this GPU's profile key, records the HBM bandwidth it measures, tunes the matmul of every benchmark shape for
every decode batch bucket, stores the winners in the SQLite profile database, then installs them on a fresh backend to show
what a host that opens the database would run.  One JSON report on stdout."""
from __future__ import annotations

import argparse
import ctypes as C
import json
import sys

from .. import backend as hb
from .. import synth
from . import plan as P
from .cost_model import CostModel, calibrate_gflops_per_thread
from .db import ProfileDb
from .tuner import TuneOptions


def measure_hbm_gbps(be: hb.CudaBackend, nbytes: int = 1 << 30, reps: int = 5) -> float:
    """Device-to-device copy bandwidth (read + write bytes over CUDA-event time), best of `reps`."""
    st = be.create_stream()
    a, b = be.allocate(nbytes, zero=False), be.allocate(nbytes, zero=False)
    e0, e1 = C.c_void_p(), C.c_void_p()
    be.lib.halo_cuda_event_create(be.ctx, C.byref(e0))
    be.lib.halo_cuda_event_create(be.ctx, C.byref(e1))
    best = 0.0
    for _ in range(reps + 1):
        be.lib.halo_cuda_event_record(be.ctx, e0, st.handle)
        be.copy(st, hb.TensorRef.of(a), hb.TensorRef.of(b), nbytes)
        be.lib.halo_cuda_event_record(be.ctx, e1, st.handle)
        ns = C.c_uint64()
        be.lib.halo_cuda_event_elapsed_ns(be.ctx, e0, e1, C.byref(ns))
        best = max(best, 2.0 * nbytes / max(ns.value, 1))
    a.free()
    b.free()
    return best


def main() -> None:
    ap = argparse.ArgumentParser(prog="python -m halo_b200.autotune")
    ap.add_argument("--db", required=True)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--shapes", default="all", choices=["all", "headline"])
    ap.add_argument("--strategy", default="exhaustive", choices=["exhaustive", "grid", "random", "heuristic"])
    ap.add_argument("--heuristic-keep", type=int, default=3)
    ap.add_argument("--random-budget", type=int, default=4)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()
    be = hb.CudaBackend(args.device)
    key = P.profile_key_of(be)
    db = ProfileDb(args.db)
    gbps = measure_hbm_gbps(be)
    db.record_tier_bandwidth(key, tier="vram", processor="gpu", label="hbm3e device-to-device copy (measured)", threads=be.info().sm_count,
                             buffer_bytes=1 << 30, read_gbps=gbps, write_gbps=gbps, copy_gbps=gbps)
    shapes = P.HEADLINE_SHAPES if args.shapes == "all" else P.HEADLINE_SHAPES[:1]
    opts = TuneOptions(strategy=args.strategy, heuristic_keep=args.heuristic_keep, random_budget=args.random_budget, seed=args.seed)
    if args.strategy == "heuristic":
        # per-SM throughput calibrated on this backend's own kernel: one tuned run of the headline shape
        probe = P.tune_shapes(be, db, key, P.HEADLINE_SHAPES[:1], (("1", 1, 1),), TuneOptions())[P.HEADLINE_SHAPES[0]]["1"]
        n, k = P.HEADLINE_SHAPES[0][1], P.HEADLINE_SHAPES[0][2]
        gf = calibrate_gflops_per_thread(2.0 * n * k, probe.winner_median_ns or 1e4, be.info().sm_count)
        opts.cost_model = CostModel.from_measurements([{"tier": "vram", "threads": be.info().sm_count, "read_gbps": gbps}], gf, launch_ns=2500.0)
    results = P.tune_shapes(be, db, key, shapes, options=opts)
    db.close()
    fresh = hb.CudaBackend(args.device)
    choices = P.install(fresh, ProfileDb(args.db, readonly=True), key, shapes)
    names = {i: n for i, n, _ in be.variants(3)}
    report = {"schema": "halo_b200.tune.report/1", "db": args.db, "hbm_copy_gbps": gbps, "strategy": args.strategy,
              "ops": [{"wtype": synth.TYPE_NAMES[s[0]], "rows": s[1], "cols": s[2], "bucket": b,
                       "winner": names.get(r.winner.get("variant")) if r.winner else None, "median_ns": r.winner_median_ns,
                       "candidates": [c.to_json() for c in r.candidates]} for s, per in results.items() for b, r in per.items()],
              "installed": [{"wtype": synth.TYPE_NAMES[c.wtype], "rows": c.rows, "cols": c.cols, "bucket": c.bucket,
                             "variant": names.get(c.variant), "source": c.source} for c in choices]}
    json.dump(report, sys.stdout)
    sys.stdout.write("\n")


if __name__ == "__main__":
    main()
