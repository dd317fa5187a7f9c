"""The matmul of the cuda backend as a tunable operator: candidates are the registered kernel variants, a run returns
device nanoseconds from CUDA events around back-to-back launches that cycle through several copies of the weights (so
that a 50 MB matrix is streamed from HBM, not from L2), and validation compares each candidate with the bit-exact variant
on the same bytes (tolerance 1e-3 relative max error, the contract of the path)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .. import backend as hb
from .. import capi, synth
from .candidate import Candidate
from .key import OpKey


class CudaGemvTunable:
    backend = "cuda"

    def __init__(self, be: hb.CudaBackend, wtype: int, rows: int, cols: int, n_vec: int, bucket: str, *, allow_gemm: bool = False,
                 copies: int | None = None, launches_per_run: int = 8, seed: int = 0, only_family: int | None = None):
        """only_family: offer only the variants of one numerics family (the decode buckets of a shape must share the family of
        its single-row winner, include/halo/backend/backend.h:300-304)."""
        self.only_family = only_family
        self.be, self.wtype, self.rows, self.cols, self.n_vec, self.allow_gemm = be, wtype, rows, cols, n_vec, allow_gemm
        self.key = OpKey.matmul(bucket, cols, rows, synth.TYPE_NAMES[wtype])
        self.st = be.create_stream()
        w = synth.quant_weights(wtype, rows, cols, seed, 1)
        wbytes = w.nbytes
        if copies is None:  # enough distinct copies to exceed the 126 MB L2 about three times
            copies = max(1, min(16, int(3 * 126e6 // max(wbytes, 1)) + 1))
        self.launches = max(launches_per_run, copies)
        self.wb = [be.import_host_readonly(w.reshape(-1)) for _ in range(copies)]
        self.wr = []  # the same matrices in the repacked layout, where the type has one (read by the repacked variants only)
        if wtype in (synth.Q6_K, synth.Q8_0, synth.Q4_0) and cols % 256 == 0:
            self.wr = [be.repack(self.st, wtype, hb.TensorRef.of(b), rows, cols) for b in self.wb]
        self.xb = be.import_host_readonly(synth.activations(n_vec, cols, seed, 2))
        self.yb = be.allocate(n_vec * rows * 4)
        self.yref = be.allocate(n_vec * rows * 4)
        self._ref = None
        lib, ctx = be.lib, be.ctx
        self.e0, self.e1 = C.c_void_p(), C.c_void_p()
        lib.halo_cuda_event_create(ctx, C.byref(self.e0))
        lib.halo_cuda_event_create(ctx, C.byref(self.e1))
        self.family = {i: fam for i, _, fam in be.variants(capi.OP_GEMV)}

    def _args(self, i: int, ybuf, variant: int) -> hb.GemvArgs:
        wbuf = self.wr[i] if variant in capi.REPACKED_VARIANTS else self.wb[i]
        return hb.GemvArgs(self.wtype, hb.TensorRef.of(wbuf), hb.TensorRef.of(self.xb), hb.TensorRef.of(ybuf), self.rows, self.cols,
                           self.n_vec, variant, allow_gemm=self.allow_gemm)

    def candidates(self) -> list[Candidate]:
        out = []
        for vid, name, _fam in self.be.variants(capi.OP_GEMV):
            if name.startswith("gemm_") and not self.allow_gemm:
                continue  # the fp16 GEMM numerics need the caller's consent (GemvArgs::allow_gemm)
            if name == "gemv_mma_m1" and self.n_vec > 4:
                continue  # one launch per row: not a candidate for wide batches
            if vid in capi.REPACKED_VARIANTS and not self.wr:
                continue  # no repacked layout for this type
            if self.only_family is not None and _fam != self.only_family:
                continue
            out.append(Candidate.of(variant=vid))
        return out

    def close(self) -> None:
        """Gives the operator's device buffers back."""
        self.st.wait()
        for b in self.wb + self.wr + [self.xb, self.yb, self.yref]:
            b.free()
        self.wb, self.wr = [], []

    def cost(self, c: Candidate):
        """What a candidate does, for the cost model: the reference's own accounting of a matmul
        (include/halo/backends/cpu/traffic.h:94-99: weight bytes + 4 M K read, 4 M N written; 2 M N K flops), one launch, every SM."""
        from .cost_model import CostInputs
        rb = synth.row_bytes(self.wtype, self.cols)
        nbytes = self.rows * rb + 4 * self.n_vec * self.cols + 4 * self.n_vec * self.rows
        return CostInputs(flops=2.0 * self.n_vec * self.rows * self.cols, bytes=nbytes, tier="vram", parallelism=self.be.info().sm_count,
                          launches=self.n_vec if c.get("variant") == capi.GEMV_MMA_M1 else 1)

    def _reference(self) -> np.ndarray:
        if self._ref is None:
            self.be.gemv(self.st, self._args(0, self.yref, capi.GEMV_EXACT8))
            ref = np.empty((self.n_vec, self.rows), np.float32)
            self.be.download(self.st, hb.TensorRef.of(self.yref), ref)
            self.st.wait()
            self._ref = ref
        return self._ref

    def validate(self, c: Candidate) -> bool:
        try:
            self.be.gemv(self.st, self._args(0, self.yb, c.get("variant")))
        except hb.HaloError:
            return False  # the variant does not take this type / shape
        y = np.empty((self.n_vec, self.rows), np.float32)
        self.be.download(self.st, hb.TensorRef.of(self.yb), y)
        self.st.wait()
        ref = self._reference()
        scale = float(np.max(np.abs(ref))) or 1.0
        return bool(np.all(np.isfinite(y)) and float(np.max(np.abs(y - ref))) <= 1e-3 * scale)

    def run(self, c: Candidate) -> float:
        lib, ctx, st = self.be.lib, self.be.ctx, self.st
        structs = [self.be._gemv_struct(self._args(i % len(self.wb), self.yb, c.get("variant")), "MATMUL", False)
                   for i in range(self.launches)]
        lib.halo_cuda_event_record(ctx, self.e0, st.handle)
        for g in structs:
            rc = lib.halo_cuda_gemv(ctx, C.byref(g), st.handle)
            if rc != 0:
                raise hb.HaloError(rc, capi.last_error())
        lib.halo_cuda_event_record(ctx, self.e1, st.handle)
        ns = C.c_uint64()
        rc = lib.halo_cuda_event_elapsed_ns(ctx, self.e0, self.e1, C.byref(ns))
        if rc != 0:
            raise hb.HaloError(rc, capi.last_error())
        return ns.value / self.launches
