"""Times the decode path over a grid of shapes: `python -m halo_b200.sweep [--types q4_k,q8_0] [--n 1024,32768] [--k 4096,17408] [--m 1,8]`.

Every (type, N, K) is loaded the way a loader of this backend loads it (Q4_K raw, the other types repacked once) and timed at each batch size
through `halo_cuda_gemv` with the variant the backend names for it, over enough distinct weight copies to exceed L2, back to back on one
stream with CUDA events.  One line per shape: microseconds, the share of the measured HBM rate the weight bytes make, and the time relative
to the first batch size -- a batch that costs much more than a single row, or a shape far below its neighbours, is a partition or tiling
cliff (the partition and the token tiles are functions of the shape: halo_cuda_gemv_plan_i8, halo_cuda_gemv_tiles_i8)."""
from __future__ import annotations

import argparse
import ctypes as C
import json
import pathlib
import sys
import time

import numpy as np

from . import backend as hb
from . import capi, synth


def hbm_gbs() -> float:
    """The measured copy rate of the GPU where a MEASURED_PEAKS.json beside the package records one (key hbm_gbs), else an earlier
    measurement of the same part."""
    p = pathlib.Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["hbm_gbs"])
    except (OSError, KeyError, ValueError):
        return 6650.0


def weights(wtype: int, rows: int, cols: int) -> np.ndarray:
    """Synthetic rows; a tall matrix repeats a 4096-row block (the kernels' time does not depend on the values)."""
    base = synth.quant_weights(wtype, min(rows, 4096), cols, 0, 1).reshape(min(rows, 4096), -1)
    return np.ascontiguousarray(np.tile(base, (-(-rows // base.shape[0]), 1))[:rows])


def time_shape(be: hb.CudaBackend, st, wtype: int, rows: int, cols: int, batches, min_bytes: float = 400e6, reps: int = 10) -> dict[int, float]:
    lib, ctx = be.lib, be.ctx
    e0, e1 = C.c_void_p(), C.c_void_p()
    lib.halo_cuda_event_create(ctx, C.byref(e0))
    lib.halo_cuda_event_create(ctx, C.byref(e1))
    w = weights(wtype, rows, cols)
    copies = max(2, min(8, int(min_bytes // w.nbytes)))
    raw = be.import_host_readonly(w.reshape(-1))
    if wtype == synth.Q4_K:
        bufs, variant = [be.import_host_readonly(w.reshape(-1)) for _ in range(copies)], 0
    else:
        bufs = [be.repack(st, wtype, hb.TensorRef.of(raw), rows, cols) for _ in range(copies)]
        variant = be.repacked_variant(wtype, cols)
    st.wait()
    out = {}
    for m in batches:
        xb = be.import_host_readonly(synth.activations(m, cols, 0, 2))
        yb = be.allocate(m * rows * 4)
        calls = [be._gemv_struct(hb.GemvArgs(wtype, hb.TensorRef.of(b), hb.TensorRef.of(xb), hb.TensorRef.of(yb), rows, cols, m, variant), "MATMUL", False)
                 for b in bufs]

        def one_pass():
            for g in calls:
                rc = lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
                if rc != 0:
                    raise hb.HaloError(rc, capi.last_error())

        one_pass()
        one_pass()
        st.wait()
        lib.halo_cuda_event_record(ctx, e0, st.handle)
        for _ in range(reps):
            one_pass()
        lib.halo_cuda_event_record(ctx, e1, st.handle)
        ns = C.c_uint64()
        lib.halo_cuda_event_elapsed_ns(ctx, e0, e1, C.byref(ns))
        out[m] = ns.value / 1e3 / (reps * copies)
        xb.free()
        yb.free()
    for b in bufs + [raw]:
        b.free()
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ints = lambda s: tuple(int(v) for v in s.split(","))  # noqa: E731
    ap.add_argument("--types", default="q4_k,q4_0,q8_0,q6_k")
    ap.add_argument("--n", type=ints, default=(1024, 4096, 8192, 32768, 128256))
    ap.add_argument("--k", type=ints, default=(2048, 4096, 5120, 8192, 14336, 17408, 28672))
    ap.add_argument("--m", type=ints, default=(1, 2, 4, 8, 16))
    ap.add_argument("--max-weights", type=float, default=1.3e9, help="skip shapes of more weights than this")
    ap.add_argument("--budget-s", type=float, default=600.0, help="stop after this many seconds")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args()
    be = hb.CudaBackend(args.device)
    st = be.create_stream()
    peak, t0 = hbm_gbs(), time.time()
    for k in args.k:
        for n in args.n:
            if n * k > args.max_weights:
                continue
            for name in args.types.split(","):
                if time.time() - t0 > args.budget_s:
                    print("time budget spent", file=sys.stderr)
                    return
                wtype = synth.TYPE_IDS[name]
                us = time_shape(be, st, wtype, n, k, args.m)
                nbytes = n * synth.row_bytes(wtype, k)
                first = us[args.m[0]]
                print(f"{name:5s} N={n:6d} K={k:6d} {nbytes / 1e6:7.1f} MB  " + "  ".join(
                    f"M={m}: {us[m]:7.1f} us ({nbytes / us[m] / 1e3 / peak * 100:3.0f} %, x{us[m] / first:4.2f})" for m in args.m), flush=True)


if __name__ == "__main__":
    main()
