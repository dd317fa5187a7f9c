"""Benchmark of the quantized weight matmul on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Metric (one JSON line on stdout): weight GB/s of the decode-shaped Q4_K matmul 17408 x 5120 at M = 1, and as
the `prefill` object the TFLOP/s of the same weights at M = 2048.  A step is one pass of Backend::gemv over
COPIES distinct copies of the weight matrix (COPIES x 50 MB, several times the 126 MB L2, so every launch
streams its weights from HBM).  `value` times launches on inputs resident in HBM; `e2e` times the same pass
through the backend's public calls with host buffers (every step copies its x rows up from pinned memory and its y
rows down; two steps are in flight on two streams, so the copies of one overlap the matmuls of the other).
`--impl reference` times the reference's own CPU backend on the same workload with all host threads.
Under torchrun each rank owns one GPU and an equal column shard of an N-times-wider projection (weak scaling,
no collective on the data path: a column split needs none).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_ROWS, K_COLS = 17408, 5120
COPIES = 16
PREFILL_M = 2048
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel on this shape (one ncu capture)
NCU_DRAM_BYTES_PER_LAUNCH = 50_193_664 + 1_024  # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel (the capture summarised next to the benchmark's profiles)
FALLBACK_HBM_GBS, FALLBACK_TFLOPS = 6650.0, 1590.0


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_TFLOPS, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [v.strip() for v in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def make_inputs(seed: int):
    from halo_b200 import synth
    w = synth.quant_weights(synth.Q4_K, N_ROWS, K_COLS, seed, 1)
    x = synth.activations(1, K_COLS, seed, 2)
    return w, x


def cpu_pass(chk, w_copies, x, threads):
    """One CPU step: the gemv over every weight copy."""
    from halo_b200 import synth
    y = None
    for w in w_copies:
        y = chk.gemv(synth.Q4_K, w, x, N_ROWS, K_COLS, threads=threads)
    return y


def cpu_baseline(copies: int = 4, passes: int = 6):
    """The reference's own CPU backend on the headline workload (Q4_K 17408 x 5120, M = 1), all host threads: one warm pass over
    every copy, then `passes` timed passes (24 calls with the defaults)."""
    import oracle
    from halo_b200 import synth
    chk = oracle.best_checker()
    threads = chk.default_threads()
    w, x = make_inputs(0)
    ws = [w.copy() for _ in range(copies)]
    cpu_pass(chk, ws, x, threads)  # warm-up: the thread pool is up, every copy has been touched
    t0 = time.perf_counter()
    for _ in range(passes):
        cpu_pass(chk, ws, x, threads)
    dt = time.perf_counter() - t0
    wbytes = N_ROWS * synth.row_bytes(synth.Q4_K, K_COLS)
    return {"value": passes * copies * wbytes / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": chk.kind,
            "sample": f"{passes} passes over {copies} copies of the Q4_K {N_ROWS}x{K_COLS} matrix, M=1 ({passes * copies} calls after a warm pass)"}, dt


def cpu_baselines_other_configs():
    """The same CPU backend on a bounded sample of every other configuration (one warm call, then `calls` timed): the down-projection
    shapes at M = 1, 4, 8; the prefill GEMM at M = 2048 on a 512-row slice of N; one Gated-DeltaNet and one GQA layer of the token
    sweep at M = 1; the Q4_0 FFN shape and an 8192-row slab of the output head at M = 16."""
    import oracle
    from halo_b200 import synth
    chk = oracle.best_checker()
    threads = chk.default_threads()
    out = []

    def timed(wtype, n, k, m, calls):
        w = synth.quant_weights(wtype, n, k, 3, 1)
        x = synth.activations(m, k, 3, 2)
        chk.gemv(wtype, w, x, n, k, threads=threads)
        t0 = time.perf_counter()
        for _ in range(calls):
            chk.gemv(wtype, w, x, n, k, threads=threads)
        return (time.perf_counter() - t0) / calls, n * synth.row_bytes(wtype, k)

    for name, wtype in (("cfg1 q6_k down", synth.Q6_K), ("cfg1 q8_0 down", synth.Q8_0)):
        for m in (1, 4, 8):
            dt, nbytes = timed(wtype, 5120, 17408, m, 4)
            out.append({"config": name, "m": m, "value": nbytes / dt / 1e9, "unit": "GB/s", "sample": "4 calls, full shape 5120 x 17408"})
    dt, _ = timed(synth.Q4_K, 512, 5120, PREFILL_M, 2)
    out.append({"config": "cfg2 q4_k prefill", "m": PREFILL_M, "value": 2.0 * PREFILL_M * 512 * 5120 / dt / 1e12, "unit": "TFLOP/s",
                "sample": "2 calls on a 512-row slice of N = 17408 (the CPU's time is linear in N)"})
    gdn, gqa = sweep_layers()
    for name, layer in (("cfg3 one GDN layer", gdn), ("cfg3 one GQA layer", gqa)):
        secs = nbytes = 0.0
        for members, wtype, k, _ in layer:
            for _, n in members:
                dt, b = timed(wtype, n, k, 1, 2)
                secs, nbytes = secs + dt, nbytes + b
        out.append({"config": name, "m": 1, "value": nbytes / secs / 1e9, "unit": "GB/s", "sample": "every projection of the layer, 2 calls each"})
    dt, nbytes = timed(synth.Q4_0, 17408, 5120, 16, 3)
    out.append({"config": "cfg4 q4_0 ffn gate / up", "m": 16, "value": nbytes / dt / 1e9, "unit": "GB/s", "sample": "3 calls, full shape"})
    dt, nbytes = timed(synth.Q4_0, 8192, 5120, 16, 3)
    out.append({"config": "cfg4 q4_0 head", "m": 16, "value": nbytes / dt / 1e9, "unit": "GB/s",
                "sample": "3 calls on one 8192-row slab of the 151936-row head (the CPU walks the head slab by slab)"})
    return {"cores": threads, "kind": chk.kind, "rows": out}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from halo_b200 import synth
    copies = 4  # bounded sample: 4 distinct 50 MB matrices already exceed the host's last-level cache
    import oracle
    chk = oracle.best_checker()
    threads = chk.default_threads()
    w, x = make_inputs(0)
    ws = [w.copy() for _ in range(copies)]
    for _ in range(max(args.warmup, 1)):
        cpu_pass(chk, ws, x, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_pass(chk, ws, x, threads)
    dt = time.perf_counter() - t0
    wbytes = N_ROWS * synth.row_bytes(synth.Q4_K, K_COLS)
    value = args.steps * copies * wbytes / dt / 1e9
    line = {"impl": "reference", "metric": "q4_k_mul_mat_weight_gbs_m1", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"cfg0: Q4_K mul_mat N={N_ROWS} K={K_COLS} M=1, {copies} weight copies per step (bounded sample)"},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": chk.kind,
                             "sample": f"{args.steps} steps x {copies} calls on host memory"},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# The per-token decode weight sweep: a 64-layer hybrid stack (48 Gated-DeltaNet + 16 GQA layers, hidden 5120, FFN 17408) in
# which every projection is a matmul.  Projections that read the same x are one grouped operand (the reference's fused qkv,
# beta|alpha and gate|up operands, src/models/qwen35.cpp:79-96, 220-253): one launch instead of one per member.
#   (members [(name, N)], type, K, split)
def sweep_layers():
    from halo_b200 import synth
    q4, q6 = synth.Q4_K, synth.Q6_K
    ffn = [([("ffn_gate", 17408), ("ffn_up", 17408)], q4, 5120, "column"), ([("ffn_down", 5120)], q6, 17408, "row")]
    gdn = [([("gdn_qkv", 10240), ("gdn_z", 6144), ("gdn_beta", 48), ("gdn_alpha", 48)], q4, 5120, "column"), ([("gdn_out", 5120)], q4, 6144, "row")] + ffn
    gqa = [([("attn_q", 5120), ("attn_k", 1024)], q4, 5120, "column"), ([("attn_v", 1024)], q6, 5120, "column"),
           ([("attn_o", 5120)], q4, 5120, "row")] + ffn
    return gdn, gqa


def time_token_pass(projs, xs_of, m: int, steps: int, world: int):
    """One x row set through every projection, `steps` times: ms per pass (max over ranks) and whether the pass ran as a CUDA graph."""
    import torch
    import torch.distributed as dist
    xs = xs_of(m)

    def one_token():
        for p in projs:
            p(xs[p.full_cols])  # the projection cuts its own K range out of a full-width x (row split)

    for _ in range(3):
        one_token()
    torch.cuda.synchronize()
    # The token pass is launch-bound when issued from Python: capture it once as a CUDA graph and replay it.
    replay, graphed = one_token, False
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            one_token()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                one_token()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        replay, graphed = graph.replay, True
    except Exception as exc:  # noqa: BLE001 - fall back to eager launches and say so
        sys.stderr.write(f"tp_sweep: CUDA graph capture failed ({exc!r}); timing eager launches\n")
        torch.cuda.synchronize()
    for _ in range(2):
        replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, graphed


def tp_sweep(local_rank: int, rank: int, world: int, steps: int, n_layers: int = 64):
    """The full per-token decode weight sweep, tensor-parallel over `world` GPUs: column split for the grouped qkv / gate|up
    operands, row split for out / o / down.  With more than one GPU the row splits are timed twice: partial products + NCCL
    all-reduce, and the matmul kernel's peer-memory epilogue (rows pushed to the peers over NVLink, added by a small kernel).
    Every distinct projection is also checked against the single-GPU product of the same weights (largest relative error)."""
    import torch
    import torch.distributed as dist

    from halo_b200 import synth, tp, tp_cuda
    rt = tp_cuda.CudaTp(local_rank, rank, world)
    one = tp_cuda.CudaTp(local_rank, 0, 1) if world > 1 else None
    gdn, gqa = sweep_layers()
    host, loaded, total_bytes, launches = {}, [], 0, 0

    def host_w(wtype, n, k):
        key = (wtype, n, k)
        if key not in host:
            host[key] = synth.quant_weights(wtype, n, k, 7, len(host) + 1)
        return host[key]

    if world > 1:
        rt.enable_peer_reduce(4 * 5120)  # the widest row-split result: 4 x rows of 5120
    # every layer owns its weights in HBM (no reuse through L2); (shard, buffer, variant) are shared by the two reduction modes
    for li in range(n_layers):
        for members, wtype, k, mode in (gqa if li % 4 == 3 else gdn):
            ws = [(host_w(wtype, n, k), n) for _, n in members]
            if mode == "column":
                proj, _ = rt.load_group(wtype, ws, k)
            else:
                proj = rt.load(wtype, ws[0][0], ws[0][1], k, "row")
            loaded.append((proj.shard, proj.buf, proj.variant, k))
            total_bytes += sum(n * synth.row_bytes(wtype, k) for _, n in members)
            launches += 1

    def projections(fused: bool):
        keep, rt.peers = rt.peers, (rt.peers if fused else None)
        out = []
        for sh, buf, variant, k in loaded:
            p = rt._projection(sh, buf, variant)
            p.full_cols = k
            out.append(p)
        rt.peers = keep
        return out

    def xs_of(m):
        torch.manual_seed(1234 + m)
        return {k: torch.randn((m, k), device="cuda", dtype=torch.float32) for k in (5120, 6144, 17408)}

    out = {}
    modes = (("nccl", False), ("peer_epilogue", True)) if world > 1 else (("none", False),)
    for how, fused in modes:
        projs = projections(fused)
        for m in (1, 4):
            ms, graphed = time_token_pass(projs, xs_of, m, steps, world)
            out[f"m{m}" if how != "peer_epilogue" else f"m{m}_peer_epilogue"] = {
                "ms_per_token": ms, "weight_gbs": total_bytes / (ms * 1e-3) / 1e9, "launches_per_token": launches,
                "row_split_reduction": how, "cuda_graph": graphed}
    # parity: the layer-0 instance of every distinct projection against the single-GPU product of the same weights
    parity = {}
    if world > 1:
        xs = xs_of(4)
        seen = set()
        for how, fused in modes:
            worst = 0.0
            projs = projections(fused)
            idx = 0
            for li in range(min(n_layers, 4)):
                for members, wtype, k, mode in (gqa if li % 4 == 3 else gdn):
                    key = (how, tuple(members), k)
                    p = projs[idx]
                    idx += 1
                    if key in seen:
                        continue
                    seen.add(key)
                    y = p(xs[k])
                    at = 0
                    for (name, n) in members:
                        full = one.load(wtype, host_w(wtype, n, k), n, k, "column")(xs[k])
                        if mode == "row":
                            got, want = y, full
                        else:
                            n0, n1 = tp.column_ranges(n, world)[rank]
                            got, want = y[:, at:at + (n1 - n0)], full[:, n0:n1]
                            at += n1 - n0
                        if want.numel():
                            worst = max(worst, float((got - want).abs().max() / full.abs().max()))
                        one._weights.popitem()[1].free()
            t = torch.tensor([worst], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            parity[how] = float(t.item())
    out["parity_rel_err_vs_single_gpu"] = parity
    out["workload"] = (f"cfg3: {n_layers} layers ({n_layers - n_layers // 4} GDN + {n_layers // 4} GQA), {total_bytes / 1e9:.2f} GB of Q4_K / Q6_K "
                       f"weights per token, tp={world}: column split of the grouped qkv / gate|up operands, row split + reduction out / o / down")
    out["scaling"] = "strong"
    for _, buf, _, _ in loaded:
        buf.free()
    rt.close()
    return out


def decode_shapes(be, st, rank: int, world: int, reps: int):
    """The other decode-shaped configurations, one line each: the Q6_K / Q8_0 down projection 5120 x 17408 at M = 1, 4, 8, and the
    Q4_0 MTP-head layer at M = 16 (eh_proj, q / k / v / o, gate / up / down, and the vocabulary-split LM head -- matmul + argmax -- with
    an all-gather of the logits).  Weights of these three types are repacked once at load, like any loader of this backend does; a
    step cycles enough distinct weight copies to exceed L2.  Timed with CUDA events on the launching stream."""
    import torch
    import torch.distributed as dist

    from halo_b200 import backend as hb
    from halo_b200 import capi, synth
    lib, ctx = be.lib, be.ctx
    pk = peaks()
    vocab = 151936
    cases = [("cfg1 q6_k down", synth.Q6_K, 5120, 17408, (1, 4, 8), False), ("cfg1 q8_0 down", synth.Q8_0, 5120, 17408, (1, 4, 8), False),
             ("cfg4 q4_0 eh_proj", synth.Q4_0, 5120, 10240, (16,), False), ("cfg4 q4_0 attn q / o", synth.Q4_0, 5120, 5120, (16,), False),
             ("cfg4 q4_0 attn k / v", synth.Q4_0, 1024, 5120, (16,), False), ("cfg4 q4_0 ffn gate / up", synth.Q4_0, 17408, 5120, (16,), False),
             ("cfg4 q4_0 ffn down", synth.Q4_0, 5120, 17408, (16,), False),
             # the same layer with the projections that read one x held as ONE operand, as the reference's models hold them
             # (src/models/qwen35.cpp:79-96, 220-253) and the decode sweep below loads them: one launch each
             ("cfg4 q4_0 attn q|k|v as one operand", synth.Q4_0, 5120 + 1024 + 1024, 5120, (16,), False),
             ("cfg4 q4_0 ffn gate|up as one operand", synth.Q4_0, 2 * 17408, 5120, (16,), False),
             ("cfg4 q4_0 lm_head (matmul + argmax), vocab split", synth.Q4_0, vocab // world, 5120, (16,), True)]
    out = []
    e0, e1 = C.c_void_p(), C.c_void_p()
    lib.halo_cuda_event_create(ctx, C.byref(e0))
    lib.halo_cuda_event_create(ctx, C.byref(e1))
    for name, wtype, n, k, ms_list, gather in cases:
        w = synth.quant_weights(wtype, n, k, 11 + rank, 1)
        wbytes = w.nbytes
        copies = max(2, min(128, -(-int(300e6) // wbytes)))  # at least 300 MB of distinct weights per cycle: more than twice L2
        raw = be.import_host_readonly(w.reshape(-1))
        packed = [be.repack(st, wtype, hb.TensorRef.of(raw), n, k) for _ in range(copies)]
        st.wait()
        variant = be.repacked_variant(wtype, k)  # what a loader passes with a repacked tensor of this type and K
        for m in ms_list:
            x = synth.activations(m, k, 11 + rank, 2)
            xb = be.import_host_readonly(x)
            yb = be.allocate(m * n * 4)
            structs = [be._gemv_struct(hb.GemvArgs(wtype, hb.TensorRef.of(b), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m, variant),
                                       "MATMUL", False) for b in packed]
            heads = []
            if gather:  # the LM head proper: the matmul over this rank's vocabulary shard, the argmax of its rows, the shard's row offset
                resb = be.allocate(m * 12)
                for g in structs:
                    h = capi.LmHead()
                    h.gemv, h.result, h.ids, h.valid_rows, h.row_offset = g, resb.ptr, None, 0, rank * n
                    heads.append(h)
            yt = torch.empty((m, n), dtype=torch.float32, device="cuda")
            full = torch.empty((world, m, n), dtype=torch.float32, device="cuda") if gather and world > 1 else None
            ts = torch.cuda.ExternalStream(st.handle)

            def one():
                for i, g in enumerate(structs):
                    rc = lib.halo_cuda_lm_head(ctx, C.byref(heads[i]), st.handle) if heads else lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
                    if rc != 0:
                        raise hb.HaloError(rc, capi.last_error())
                    if full is not None:  # the logits of every shard on every rank
                        lib.halo_cuda_memcpy_d2d_async(ctx, C.c_void_p(yt.data_ptr()), g.y, m * n * 4, st.handle)
                        with torch.cuda.stream(ts):
                            dist.all_gather_into_tensor(full, yt)

            for _ in range(3):
                one()
            st.wait()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            lib.halo_cuda_event_record(ctx, e0, st.handle)
            for _ in range(reps):
                one()
            lib.halo_cuda_event_record(ctx, e1, st.handle)
            st.wait()
            torch.cuda.synchronize()
            ns = C.c_uint64()
            lib.halo_cuda_event_elapsed_ns(ctx, e0, e1, C.byref(ns))
            us = ns.value / 1e3 / (reps * copies)
            if world > 1:
                t = torch.tensor([us], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                us = float(t.item())
            # parity of what was timed: against the exact-order kernel on the raw rows
            y = np.empty((m, n), np.float32)
            be.download(st, hb.TensorRef.of(yb), y)
            be.gemv(st, hb.GemvArgs(wtype, hb.TensorRef.of(raw), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m, capi.GEMV_EXACT8))
            ye = np.empty((m, n), np.float32)
            be.download(st, hb.TensorRef.of(yb), ye)
            st.wait()
            shards = world if gather else 1  # the FFN / down shapes are per-GPU work (weak), the head is one job split over the ranks
            gbs = shards * wbytes / (us * 1e-6) / 1e9
            out.append({"shape": name, "wtype": synth.TYPE_NAMES[wtype], "variant": variant, "rows_per_gpu": n, "cols": k, "m": m, "us_per_call": us,
                        "weight_gbs": gbs, "frac_of_hbm_per_gpu": gbs / shards / pk["hbm_gbs"], "all_gather": bool(full is not None),
                        "rel_err_vs_exact": float(np.max(np.abs(y - ye)) / np.max(np.abs(ye)))})
            xb.free()
            yb.free()
            if heads:
                resb.free()
        for b in packed:
            b.free()
        raw.free()
    return out


def fused_norm_leg(be, st, reps: int = 20, copies: int = 8):
    """The matmul with the fused input norm (GemvArgs::norm_w) beside the plain matmul of the same shape: config 0 and the Q6_K
    shape of config 1, one x row, `copies` distinct weight copies cycled (> L2), CUDA events on the launching stream."""
    import numpy as np

    from halo_b200 import backend as hb
    from halo_b200 import capi, synth

    lib, ctx = be.lib, be.ctx
    e0, e1 = C.c_void_p(), C.c_void_p()
    lib.halo_cuda_event_create(ctx, C.byref(e0))
    lib.halo_cuda_event_create(ctx, C.byref(e1))
    out = []
    for name, t, n, k, variant in (("cfg0 q4_k", synth.Q4_K, N_ROWS, K_COLS, 0), ("cfg1 q6_k down", synth.Q6_K, 5120, 17408, be.repacked_variant(synth.Q6_K, 17408))):
        w = synth.quant_weights(t, n, k, 0, 1)
        bufs = []
        for _ in range(copies):
            b = be.import_host_readonly(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
            if variant in capi.REPACKED_VARIANTS:
                p = be.repack(st, t, hb.TensorRef.of(b), n, k)
                st.wait()
                b.free()
                b = p
            bufs.append(b)
        xb = be.import_host_readonly(synth.activations(1, k, 0, 2))
        nw = be.import_host_readonly(np.full(k, 1.25, np.float32))
        yb = be.allocate(n * 4)
        row = {"shape": name, "rows": n, "cols": k, "m": 1}
        for key, fused in (("us_plain", False), ("us_fused_norm", True)):
            args = [hb.GemvArgs(t, hb.TensorRef.of(b), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, 1, variant) for b in bufs]
            if fused:
                for a in args:
                    a.norm_w = hb.TensorRef.of(nw)
            for a in args:
                be.gemv(st, a)
            st.wait()
            lib.halo_cuda_event_record(ctx, e0, st.handle)
            for _ in range(reps):
                for a in args:
                    be.gemv(st, a)
            lib.halo_cuda_event_record(ctx, e1, st.handle)
            st.wait()
            ns = C.c_uint64()
            lib.halo_cuda_event_elapsed_ns(ctx, e0, e1, C.byref(ns))
            row[key] = ns.value / 1e3 / (reps * copies)
        # what the fusion replaces: a separate RMS-norm kernel in front of the plain matmul, on the same stream (the norm is
        # torch's own rms_norm kernel, a library stand-in for the operator this backend does not have)
        import torch
        import torch.nn.functional as F
        ts = torch.cuda.ExternalStream(st.handle)
        with torch.cuda.stream(ts):
            xt = torch.from_numpy(synth.activations(1, k, 0, 2)).to("cuda")
            wt = torch.full((k,), 1.25, device="cuda", dtype=torch.float32)
            structs = [be._gemv_struct(hb.GemvArgs(t, hb.TensorRef.of(b), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, 1, variant), "MATMUL", False)
                       for b in bufs]

            def unfused():
                for g in structs:
                    xn = F.rms_norm(xt, (k,), wt, 1e-6)
                    g.x = xn.data_ptr()
                    rc = lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
                    if rc != 0:
                        raise hb.HaloError(rc, capi.last_error())

            unfused()
            st.wait()
            lib.halo_cuda_event_record(ctx, e0, st.handle)
            for _ in range(reps):
                unfused()
            lib.halo_cuda_event_record(ctx, e1, st.handle)
            st.wait()
        ns = C.c_uint64()
        lib.halo_cuda_event_elapsed_ns(ctx, e0, e1, C.byref(ns))
        row["us_rms_norm_kernel_then_plain"] = ns.value / 1e3 / (reps * copies)
        out.append(row)
        for b in bufs + [xb, nw, yb]:
            b.free()
    return out


def raw_rows_leg(be, st, reps: int = 10):
    """What plain Backend::gemv gives on RAW Q6_K / Q8_0 / Q4_0 rows (no repacking loader): variant 0 resolves to gemv_warp_f32
    there.  The FFN down shape of config 1 at M = 1 and 8, the gate / up shape of config 4 at M = 16; >= 300 MB of weight copies
    cycled, CUDA events on the launching stream."""
    from halo_b200 import backend as hb
    from halo_b200 import capi, synth

    lib, ctx = be.lib, be.ctx
    pk = peaks()
    names = {i: n for i, n, _ in be.variants(capi.OP_GEMV)}
    e0, e1 = C.c_void_p(), C.c_void_p()
    lib.halo_cuda_event_create(ctx, C.byref(e0))
    lib.halo_cuda_event_create(ctx, C.byref(e1))
    out = []
    for name, t, n, k, ms_list in (("cfg1 q6_k down", synth.Q6_K, 5120, 17408, (1, 8)), ("cfg1 q8_0 down", synth.Q8_0, 5120, 17408, (1, 8)),
                                   ("cfg4 q4_0 ffn gate / up", synth.Q4_0, 17408, 5120, (16,))):
        w = synth.quant_weights(t, n, k, 31, 1)
        copies = max(2, -(-int(300e6) // w.nbytes))
        bufs = [be.import_host_readonly(w.reshape(-1)) for _ in range(copies)]
        for m in ms_list:
            xb = be.import_host_readonly(synth.activations(m, k, 31, 2))
            yb = be.allocate(m * n * 4)
            args = [hb.GemvArgs(t, hb.TensorRef.of(b), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m, 0) for b in bufs]
            structs = [be._gemv_struct(a, "MATMUL", False) for a in args]
            ran = be.resolve_variant(args[0])
            for g in structs:
                lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
            st.wait()
            lib.halo_cuda_event_record(ctx, e0, st.handle)
            for _ in range(reps):
                for g in structs:
                    lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
            lib.halo_cuda_event_record(ctx, e1, st.handle)
            st.wait()
            ns = C.c_uint64()
            lib.halo_cuda_event_elapsed_ns(ctx, e0, e1, C.byref(ns))
            us = ns.value / 1e3 / (reps * copies)
            out.append({"shape": name, "m": m, "variant": names.get(ran, str(ran)), "us_per_call": us, "weight_gbs": w.nbytes / us / 1e3,
                        "frac_of_hbm": w.nbytes / us / 1e3 / pk["hbm_gbs"]})
            xb.free()
            yb.free()
        for b in bufs:
            b.free()
    return out


def prefill_repacked_leg(be, st, reps: int = 5):
    """The prefill GEMM over repacked Q6_K / Q8_0 / Q4_0 rows at M = 2048: the FFN down shape of config 1 in Q6_K and Q8_0, the
    gate / up shape of config 4 in Q4_0.  A call names the tensor's decode variant and sets allow_gemm, as a model would; each
    result carries its error against the oracle on a 64-row slice of N.  CUDA events on the launching stream."""
    import numpy as np

    import oracle
    from halo_b200 import backend as hb
    from halo_b200 import capi, synth

    lib, ctx = be.lib, be.ctx
    pk = peaks()
    names = {i: n for i, n, _ in be.variants(capi.OP_GEMV)}
    e0, e1 = C.c_void_p(), C.c_void_p()
    lib.halo_cuda_event_create(ctx, C.byref(e0))
    lib.halo_cuda_event_create(ctx, C.byref(e1))
    chk = oracle.best_checker()
    m, out = 2048, []
    for name, t, n, k in (("cfg1 q6_k down", synth.Q6_K, 5120, 17408), ("cfg1 q8_0 down", synth.Q8_0, 5120, 17408),
                          ("cfg4 q4_0 ffn gate / up", synth.Q4_0, 17408, 5120)):
        w = synth.quant_weights(t, n, k, 21, 1)
        x = synth.activations(m, k, 21, 2)
        raw = be.import_host_readonly(w.reshape(-1))
        pkd = be.repack(st, t, hb.TensorRef.of(raw), n, k)
        xb = be.import_host_readonly(x)
        yb = be.allocate(m * n * 4, zero=False)
        a = hb.GemvArgs(t, hb.TensorRef.of(pkd), hb.TensorRef.of(xb), hb.TensorRef.of(yb), n, k, m, be.repacked_variant(t, k), allow_gemm=True)
        g = be._gemv_struct(a, "MATMUL", False)
        ran = be.resolve_variant(a)
        for _ in range(2):
            if lib.halo_cuda_gemv(ctx, C.byref(g), st.handle) != 0:
                raise hb.HaloError(-1, capi.last_error())
        st.wait()
        lib.halo_cuda_event_record(ctx, e0, st.handle)
        for _ in range(reps):
            lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
        lib.halo_cuda_event_record(ctx, e1, st.handle)
        st.wait()
        ns = C.c_uint64()
        lib.halo_cuda_event_elapsed_ns(ctx, e0, e1, C.byref(ns))
        ms = ns.value / 1e6 / reps
        y = np.empty((m, n), np.float32)
        be.download(st, hb.TensorRef.of(yb), y)
        st.wait()
        n_slice = 64
        ref = chk.gemv(t, w.reshape(n, -1)[:n_slice], x, n_slice, k)
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out.append({"shape": name, "wtype": synth.TYPE_NAMES[t], "rows": n, "cols": k, "m": m, "variant": names.get(ran, str(ran)), "ms_per_call": ms,
                    "tflops": tf, "frac_of_bf16_burst": tf / pk["bf16_tflops"],
                    "rel_err_vs_oracle": float(np.max(np.abs(y[:, :n_slice] - ref)) / np.max(np.abs(ref))),
                    "oracle_sample": f"all {m} x rows on the first {n_slice} of {n} W rows"})
        for b in (raw, pkd, xb, yb):
            b.free()
    return out


def loader_leg(be, st, rank: int, world: int, reps: int = 3):
    """File -> device: this rank's column share of the config-4 LM head (Q4_0, 151936 x 5120, 437.6 MB in all) brought from a GGUF
    file in the page cache into HBM by the loader (pinned double-buffered staging, repack on the device), beside the plain
    import of the same bytes from pageable memory.  Wall clock around call + stream wait; best of `reps`."""
    import tempfile

    import numpy as np

    from halo_b200 import capi, gguf, synth

    rows, cols, t = 151936, 5120, synth.Q4_0
    rb = synth.row_bytes(t, cols)
    raw = np.random.default_rng(rank).integers(0, 256, rows * rb, dtype=np.uint8)
    out = {"tensor": f"Q4_0 {rows} x {cols}", "file_mb": raw.size / 1e6, "split": f"column x{world}"}
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "head.gguf")
        gguf.write_gguf(path, [("output.weight", t, rows, cols, raw)], {"general.architecture": "qwen35"})
        with gguf.GgufFile.open(path) as f:
            info = f.find_tensor("output.weight")
            share = gguf.matrix_share(t, rows, cols, capi.SPLIT_COLUMN, rank, world)
            nbytes = share.rows * rb
            for name, repack in (("upload_gbs", False), ("upload_repacked_gbs", True)):
                best = float("inf")
                for _ in range(reps + 1):
                    t0 = time.perf_counter()
                    m = gguf.upload_matrix(be, st, f, info, capi.SPLIT_COLUMN, rank, world, repack=repack)
                    st.wait()
                    best = min(best, time.perf_counter() - t0)
                    m.buf.free()
                out[name] = nbytes / best / 1e9
    lo = share.row0 * rb
    best = float("inf")
    for _ in range(reps + 1):
        t0 = time.perf_counter()
        b = be.import_host_readonly(raw[lo:lo + nbytes])
        st.wait()
        best = min(best, time.perf_counter() - t0)
        b.free()
    out["import_pageable_gbs"] = nbytes / best / 1e9
    out["share_mb"] = nbytes / 1e6
    return out


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from halo_b200 import backend as hb
    from halo_b200 import capi, synth

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the matmul path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # NCCL may announce its version on stdout when it builds the communicator; the contract of this script is one JSON line
        # there, so the communicator is built (first collective) with stdout pointed at stderr
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    be = hb.CudaBackend(local_rank)
    st = be.create_stream()
    lib, ctx = be.lib, be.ctx
    if args.profile and args.shapes:
        for r in decode_shapes(be, st, rank, world, max(1, args.steps)):
            print(json.dumps(r), flush=True)
        return

    # ---- inputs: rank r holds its own column shard (distinct seed), COPIES distinct copies resident in HBM
    w, x = make_inputs(rank)
    rb = synth.row_bytes(synth.Q4_K, K_COLS)
    wbytes = N_ROWS * rb
    wbufs = [be.import_host_readonly(w.reshape(-1)) for _ in range(COPIES)]
    xb = be.import_host_readonly(x)
    ybufs = [be.allocate(N_ROWS * 4) for _ in range(COPIES)]
    calls = [hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wbufs[i]), hb.TensorRef.of(xb), hb.TensorRef.of(ybufs[i]), N_ROWS, K_COLS, 1, args.variant)
             for i in range(COPIES)]
    structs = [be._gemv_struct(a, "MATMUL", False) for a in calls]
    variant = be.resolve_variant(calls[0])
    vname = {i: n for i, n, _ in be.variants(capi.OP_GEMV)}[variant]

    # ---- which kernel runs: the autotuner's.  The headline shape is tuned into a fresh profile database (this box has none), the
    # database is reopened read-only and its winner installed as the backend's plan, as a host does at engine creation.
    kernel_choice = None
    if not args.profile and args.variant == 0:
        import tempfile

        from halo_b200.autotune import ProfileDb
        from halo_b200.autotune import plan as tune_plan
        one = (("1", 1, 1),)
        with tempfile.TemporaryDirectory() as d:
            db_path = os.path.join(d, "profile.db")
            db = ProfileDb(db_path)
            pkey = tune_plan.profile_key_of(be)
            tuned = tune_plan.tune_shapes(be, db, pkey, tune_plan.HEADLINE_SHAPES[:1], one)[tune_plan.HEADLINE_SHAPES[0]]["1"]
            db.close()
            ro = ProfileDb(db_path, readonly=True)
            ch = tune_plan.install(be, ro, pkey, tune_plan.HEADLINE_SHAPES[:1], one)[0]
            ro.close()
        names = {i: n for i, n, _ in be.variants(capi.OP_GEMV)}
        kernel_choice = {"source": ch.source, "variant": names.get(ch.variant), "strategy": "exhaustive",
                         "candidates_us": {names[r.candidate.get("variant")]: (round(r.stats["median"] / 1e3, 2) if r.measured else None)
                                           for r in tuned.candidates},
                         "rejected": {names[r.candidate.get("variant")]: r.rejected for r in tuned.candidates if r.rejected}}
        variant = be.resolve_variant(calls[0])
        vname = names[variant]

    def one_pass():
        for g in structs:
            rc = lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
            if rc != 0:
                raise hb.HaloError(rc, capi.last_error())

    def barrier():
        st.wait()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = C.c_void_p(), C.c_void_p()
        lib.halo_cuda_event_create(ctx, C.byref(e0))
        lib.halo_cuda_event_create(ctx, C.byref(e1))
        barrier()
        lib.halo_cuda_event_record(ctx, e0, st.handle)
        for _ in range(steps):
            fn()
        lib.halo_cuda_event_record(ctx, e1, st.handle)
        ns = C.c_uint64()
        rc = lib.halo_cuda_event_elapsed_ns(ctx, e0, e1, C.byref(ns))
        if rc != 0:
            raise hb.HaloError(rc, capi.last_error())
        barrier()
        ms = ns.value / 1e6
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    n_warm = args.warmup if args.profile else max(args.warmup, 3)
    for _ in range(n_warm):
        one_pass()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(one_pass, args.steps)

    # The same resident pass with its 16 independent matmuls issued alternately on two streams (informative, not the headline:
    # in a decode chain every matmul waits for the one before it).  The two streams fill each other's launch turnaround.
    two_stream = None
    if not args.profile:
        st2 = be.create_stream()
        ev0, ev1, ev2 = C.c_void_p(), C.c_void_p(), C.c_void_p()
        for e in (ev0, ev1, ev2):
            lib.halo_cuda_event_create(ctx, C.byref(e))

        def two_pass():
            for i, g in enumerate(structs):
                rc = lib.halo_cuda_gemv(ctx, C.byref(g), (st2 if i & 1 else st).handle)
                if rc != 0:
                    raise hb.HaloError(rc, capi.last_error())

        for _ in range(3):
            two_pass()
        st.wait()
        st2.wait()
        t0 = time.perf_counter()
        reps2 = max(1, args.steps // 2)
        for _ in range(reps2):
            two_pass()
        st.wait()
        st2.wait()
        us2 = (time.perf_counter() - t0) * 1e6 / (reps2 * COPIES)
        two_stream = {"us_per_launch": us2, "frac_of_hbm": (wbytes + 4 * K_COLS + 4 * N_ROWS) / us2 / 1e3 / peaks()["hbm_gbs"],
                      "timing": "wall clock around the launches of both streams and their waits"}

    # The gate and up projections of an FFN as the ONE operand a model holds them in (the reference's fused gate|up operand,
    # src/models/qwen35.cpp:220-253; the decode sweep below loads them the same way): 2 x 17408 rows read the same x row in one
    # launch, so the launch turnaround is paid once per 100 MB.  Informative, not the headline.
    grouped = None
    if not args.profile:
        n_pair, both = max(2, COPIES // 2), np.concatenate([w.reshape(-1), w.reshape(-1)])
        gbufs = [be.import_host_readonly(both) for _ in range(n_pair)]
        gy = be.allocate(2 * N_ROWS * 4)
        gstructs = [be._gemv_struct(hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(b), hb.TensorRef.of(xb), hb.TensorRef.of(gy), 2 * N_ROWS, K_COLS, 1, args.variant),
                                    "MATMUL", False) for b in gbufs]
        del both

        def grouped_pass():
            for g in gstructs:
                rc = lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
                if rc != 0:
                    raise hb.HaloError(rc, capi.last_error())

        for _ in range(3):
            grouped_pass()
        gsteps = max(1, args.steps // 2)
        gus = timed(grouped_pass, gsteps) * 1e3 / (gsteps * n_pair)
        yg2 = np.empty(2 * N_ROWS, np.float32)
        be.download(st, hb.TensorRef.of(gy), yg2)
        st.wait()
        y_one = np.empty(N_ROWS, np.float32)
        be.download(st, hb.TensorRef.of(ybufs[-1]), y_one)
        st.wait()
        grouped = {"rows": 2 * N_ROWS, "us_per_launch": gus, "us_per_projection": gus / 2,
                   "frac_of_hbm": (2 * wbytes + 4 * K_COLS + 8 * N_ROWS) / gus / 1e3 / peaks()["hbm_gbs"],
                   "rel_diff_vs_separate_launches": float(max(np.max(np.abs(yg2[:N_ROWS] - y_one)), np.max(np.abs(yg2[N_ROWS:] - y_one)))
                                                          / np.max(np.abs(y_one)))}
        for b in gbufs + [gy]:
            b.free()

    # ---- e2e: the same pass through the public calls with host buffers: the step's COPIES x rows go up from pinned memory in
    # one copy, every matmul reads its own row and writes its own y, the step's COPIES y rows come down in one copy.  As a host
    # that wants throughput would, two steps are in flight: steps alternate between two streams (each with its own pinned and
    # device buffers), and the host waits for step i - 2 before it issues step i, so the copies of one step overlap the matmuls of
    # the other.  Every step still copies its own inputs up and its own results down inside the timed region.
    lanes = []
    for _ in range(2):
        hx, hy = C.c_void_p(), C.c_void_p()
        lib.halo_cuda_host_alloc(ctx, COPIES * K_COLS * 4, C.byref(hx))
        lib.halo_cuda_host_alloc(ctx, COPIES * N_ROWS * 4, C.byref(hy))
        for i in range(COPIES):
            C.memmove(hx.value + i * K_COLS * 4, x.ctypes.data, K_COLS * 4)
        x_all = be.allocate(COPIES * K_COLS * 4)
        y_all = be.allocate(COPIES * N_ROWS * 4)
        stream = be.create_stream()
        structs_l = [be._gemv_struct(hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wbufs[i]), hb.TensorRef(x_all, i * K_COLS * 4, K_COLS * 4),
                                                 hb.TensorRef(y_all, i * N_ROWS * 4, N_ROWS * 4), N_ROWS, K_COLS, 1, args.variant), "MATMUL", False)
                     for i in range(COPIES)]
        lanes.append((stream, hx, hy, x_all, y_all, structs_l))

    def e2e_step(lane):
        stream, hx, hy, x_all, y_all, structs_l = lane
        stream.wait()  # the step issued two steps ago on this stream: its results are in host memory now
        lib.halo_cuda_memcpy_h2d_async(ctx, C.c_void_p(x_all.ptr), hx, COPIES * K_COLS * 4, stream.handle)
        for g in structs_l:
            rc = lib.halo_cuda_gemv(ctx, C.byref(g), stream.handle)
            if rc != 0:
                raise hb.HaloError(rc, capi.last_error())
        lib.halo_cuda_memcpy_d2h_async(ctx, hy, C.c_void_p(y_all.ptr), COPIES * N_ROWS * 4, stream.handle)

    def e2e_run(steps):
        for i in range(steps):
            e2e_step(lanes[i & 1])
        for lane in lanes:
            lane[0].wait()

    e2e_run(0 if args.profile else 6)
    barrier()
    t0 = time.perf_counter()
    e2e_run(2 if args.profile else args.steps)
    e2e_s = (time.perf_counter() - t0) * (args.steps / 2 if args.profile else 1)
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    # ---- parity spot check of what was timed (the last copy's y against the exact-order variant on the device)
    y_fast = np.empty(N_ROWS, np.float32)
    be.download(st, hb.TensorRef.of(ybufs[-1]), y_fast)
    exact = hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wbufs[-1]), hb.TensorRef.of(xb), hb.TensorRef.of(ybufs[0]), N_ROWS, K_COLS, 1,
                        capi.GEMV_EXACT8)
    be.gemv(st, exact)
    y_exact = np.empty(N_ROWS, np.float32)
    be.download(st, hb.TensorRef.of(ybufs[0]), y_exact)
    st.wait()
    rel_err = float(np.max(np.abs(y_fast - y_exact)) / np.max(np.abs(y_exact)))

    # ---- prefill half of the metric: the same weights at M = 2048 through the tcgen05 GEMM (allow_gemm) ----------------
    prefill = None
    if not args.profile or args.prefill:
        pm = PREFILL_M
        xp = synth.activations(pm, K_COLS, rank, 3)
        xpb = be.import_host_readonly(xp)
        ypb = be.allocate(pm * N_ROWS * 4, zero=False)
        pargs = hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wbufs[0]), hb.TensorRef.of(xpb), hb.TensorRef.of(ypb), N_ROWS, K_COLS, pm, 0,
                            allow_gemm=True)
        pstruct = be._gemv_struct(pargs, "MATMUL", False)
        pvariant = be.resolve_variant(pargs)
        psteps = max(1, min(args.steps, 30))

        def prefill_pass():
            rc = lib.halo_cuda_gemv(ctx, C.byref(pstruct), st.handle)
            if rc != 0:
                raise hb.HaloError(rc, capi.last_error())

        for _ in range(1 if args.profile else 3):
            prefill_pass()
        pms = timed(prefill_pass, psteps) / psteps
        # parity of what was timed against the oracle: all M x rows on a 128-row slice of N (the CPU's cost is linear in N)
        rel_oracle = None
        if rank == 0 and not args.profile:
            import oracle
            n_slice = 128
            y_all = np.empty((pm, N_ROWS), np.float32)
            be.download(st, hb.TensorRef.of(ypb), y_all)
            st.wait()
            ref = oracle.best_checker().gemv(synth.Q4_K, w.reshape(N_ROWS, rb)[:n_slice], xp, n_slice, K_COLS)
            rel_oracle = float(np.max(np.abs(y_all[:, :n_slice] - ref)) / np.max(np.abs(ref)))
            del y_all
        # and 8 tokens over all of N against the tensor-core skinny kernel of the fp16 family (near-fp32 accuracy)
        yg = np.empty((8, N_ROWS), np.float32)
        be.download(st, hb.TensorRef(ypb, 0, 8 * N_ROWS * 4), yg)
        chk = hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wbufs[0]), hb.TensorRef.of(xpb), hb.TensorRef.of(ypb), N_ROWS, K_COLS, 8,
                          capi.GEMV_MMA_F16X2)
        be.gemv(st, chk)
        ys = np.empty((8, N_ROWS), np.float32)
        be.download(st, hb.TensorRef(ypb, 0, 8 * N_ROWS * 4), ys)
        st.wait()
        flops = 2.0 * pm * N_ROWS * K_COLS
        tf = world * flops / (pms * 1e-3) / 1e12
        pkk = peaks()
        prefill = {"metric": "q4_k_mul_mat_tflops_m2048", "value": tf, "unit": "TFLOP/s", "ms_per_call": pms,
                   "variant": {i: n for i, n, _ in be.variants(capi.OP_GEMV)}.get(pvariant, str(pvariant)), "dtype": "f16 operands, f32 accumulate",
                   "rel_err_vs_skinny_kernel": float(np.max(np.abs(yg - ys)) / np.max(np.abs(ys))),
                   "rel_err_vs_oracle": rel_oracle, "oracle_sample": f"all {pm} x rows on the first 128 of {N_ROWS} W rows",
                   "roofline": {"bound": "tensor", "achieved": tf / world, "peak": pkk["bf16_tflops"], "unit": "TFLOP/s",
                                "frac": tf / world / pkk["bf16_tflops"], "frac_of_sustained": tf / world / pkk["bf16_tflops_sustained"],
                                "traffic": None, "peak_source": pkk["source"], "flops_per_launch": flops},
                   "l2": "operands larger than L2: W 50 MB + x 42 MB + y 143 MB per call", "gpu_launches": 2 * psteps}

        # the other two batch sizes of config 2, same weights (timed with fewer repetitions)
        by_m = [{"m": pm, "ms_per_call": pms, "tflops_per_gpu": flops / (pms * 1e-3) / 1e12}]
        if not args.profile:
            for om in (512, 4096):
                xo = be.import_host_readonly(synth.activations(om, K_COLS, rank, 4))
                yo = be.allocate(om * N_ROWS * 4, zero=False)
                ostruct = be._gemv_struct(hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wbufs[0]), hb.TensorRef.of(xo), hb.TensorRef.of(yo), N_ROWS,
                                                       K_COLS, om, 0, allow_gemm=True), "MATMUL", False)

                def other_pass(g=ostruct):
                    rc = lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
                    if rc != 0:
                        raise hb.HaloError(rc, capi.last_error())

                for _ in range(3):
                    other_pass()
                osteps = max(1, psteps // 2)
                oms = timed(other_pass, osteps) / osteps
                by_m.append({"m": om, "ms_per_call": oms, "tflops_per_gpu": 2.0 * om * N_ROWS * K_COLS / (oms * 1e-3) / 1e12})
                xo.free()
                yo.free()
        prefill["by_m"] = sorted(by_m, key=lambda r: r["m"])
        if world > 1:  # the same GEMM with N column-split over the ranks (strong scaling; no collective: each rank keeps its columns)
            n_split = N_ROWS // world
            sargs = hb.GemvArgs(synth.Q4_K, hb.TensorRef.of(wbufs[0]), hb.TensorRef.of(xpb), hb.TensorRef.of(ypb), n_split, K_COLS, pm, 0,
                                allow_gemm=True)
            sstruct = be._gemv_struct(sargs, "MATMUL", False)

            def split_pass():
                rc = lib.halo_cuda_gemv(ctx, C.byref(sstruct), st.handle)
                if rc != 0:
                    raise hb.HaloError(rc, capi.last_error())

            for _ in range(3):
                split_pass()
            sms = timed(split_pass, psteps) / psteps
            prefill["column_split"] = {"rows_per_gpu": n_split, "ms_per_call": sms, "tflops": flops / (sms * 1e-3) / 1e12, "scaling": "strong"}

    sweep = shapes = loader = fused_norm = prefill_r = raw_rows = None
    if not args.profile:
        for b in wbufs[1:] + ybufs[1:]:
            b.free()
        shapes = decode_shapes(be, st, rank, world, max(3, min(args.steps, 20)))
        sweep = tp_sweep(local_rank, rank, world, max(3, min(args.steps, 20)))
        loader = loader_leg(be, st, rank, world)
        fused_norm = fused_norm_leg(be, st) if rank == 0 else None
        prefill_r = prefill_repacked_leg(be, st) if rank == 0 else None
        raw_rows = raw_rows_leg(be, st) if rank == 0 else None
    clocks = sampler.stop() if rank == 0 else None

    launches_per_step = COPIES
    total_launches = args.steps * launches_per_step
    launch_us = ms * 1e3 / total_launches
    algo_bytes = wbytes + 4 * K_COLS + 4 * N_ROWS
    pk = peaks()
    achieved = algo_bytes / (launch_us * 1e-6) / 1e9
    value = world * args.steps * COPIES * wbytes / (ms * 1e-3) / 1e9
    e2e_value = world * args.steps * COPIES * wbytes / e2e_s / 1e9
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu = None
    if not args.profile:
        cpu = cpu_baseline()[0]
        cpu["by_config"] = cpu_baselines_other_configs()
    # compact copies of the other halves of the metric under `config` (the detailed objects follow as keys of their own)
    r3 = lambda v: None if v is None else round(float(v), 4)  # noqa: E731
    summary = {}
    if prefill is not None:
        summary["prefill_q4k_tcgen05"] = {"m2048_tflops": r3(prefill["value"]), "m2048_ms": r3(prefill["ms_per_call"]),
                                          "m2048_frac_of_bf16_burst": r3(prefill["roofline"]["frac"]),
                                          "by_m": [{"m": r["m"], "ms": r3(r["ms_per_call"]), "tflops_per_gpu": r3(r["tflops_per_gpu"])} for r in prefill["by_m"]],
                                          "column_split": prefill.get("column_split"), "rel_err_vs_oracle": prefill.get("rel_err_vs_oracle")}
    if prefill_r is not None:
        summary["prefill_repacked_tcgen05_m2048"] = [{"shape": r["shape"], "tflops": r3(r["tflops"]), "ms": r3(r["ms_per_call"]),
                                                      "rel_err_vs_oracle": r["rel_err_vs_oracle"]} for r in prefill_r]
    if shapes is not None:
        summary["decode_shapes"] = [{"shape": r["shape"], "m": r["m"], "us": r3(r["us_per_call"]), "frac_of_hbm": r3(r["frac_of_hbm_per_gpu"]),
                                     "rel_err": r["rel_err_vs_exact"]} for r in shapes]
    if raw_rows is not None:
        summary["raw_rows_default_variant"] = [{"shape": r["shape"], "m": r["m"], "variant": r["variant"], "us": r3(r["us_per_call"]),
                                                "frac_of_hbm": r3(r["frac_of_hbm"])} for r in raw_rows]
    if sweep is not None:
        summary["tp_sweep"] = {k: ({"ms": r3(v["ms_per_token"]), "gbs": r3(v["weight_gbs"]), "launches": v["launches_per_token"]} if k.startswith("m") else v)
                               for k, v in sweep.items() if k != "workload"}
    line = {
        "metric": "q4_k_mul_mat_weight_gbs_m1", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": n_warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"cfg0: Q4_K mul_mat N={N_ROWS} K={K_COLS} M=1 per GPU, {COPIES} distinct weight copies per step",
                   "variant": vname, "l2": f"inputs larger than L2: {COPIES} x {wbytes / 1e6:.1f} MB of weights cycled",
                   "parallelism": f"column split x{world}, no collective", "rel_err_vs_exact": rel_err, "kernel_choice": kernel_choice,
                   "two_streams_resident": two_stream, "gate_up_one_operand": grouped, **summary},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "traffic_source": "ncu capture of one launch of this kernel on this shape",
                     "peak_source": pk["source"], "kernel": vname, "launch_us": launch_us,
                     "algorithmic_bytes_per_launch": algo_bytes},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": COPIES * K_COLS * 4, "d2h_bytes_per_step": COPIES * N_ROWS * 4,
                "ms_per_step": e2e_s / args.steps * 1e3, "pipelining": "two steps in flight on two streams; every step copies its own x up and y down"},
        "gpu_launches": total_launches,
        "prefill": prefill,
        "prefill_repacked": prefill_r,
        "decode_shapes": shapes,
        "raw_rows_default_variant": raw_rows,
        "tp_sweep": sweep,
        "loader": loader,
        "fused_norm": fused_norm,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--copies", type=int, default=16, help="distinct weight copies cycled per step")
    ap.add_argument("--variant", type=int, default=0, help="kernel variant id (0 = what the backend selects)")
    ap.add_argument("--prefill", action="store_true", help="with --profile: also run the M = 2048 GEMM")
    ap.add_argument("--profile", action="store_true", help="small run for ncu: no CPU baseline, no e2e leg, warm-up as given")
    ap.add_argument("--shapes", action="store_true", help="with --profile: run only the config-1 / config-4 decode shapes (1 GPU)")
    args = ap.parse_args()
    globals()["COPIES"] = args.copies
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
