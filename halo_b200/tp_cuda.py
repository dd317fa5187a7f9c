"""The tensor-parallel projections of tp.py on the cuda backend: torch tensors for activations, NCCL for the row split.

One process per GPU.  Kernels are launched on torch's current stream, so an all-reduce issued through
torch.distributed right after a projection is ordered behind it without extra synchronisation.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import backend as hb
from . import capi, synth, tp


class CudaTp:
    def __init__(self, device: int, rank: int, world: int):
        self.be = hb.CudaBackend(device)
        self.rank, self.world = rank, world
        self.device = torch.device("cuda", device)
        self._weights: dict[int, hb.Buffer] = {}

    def stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def load(self, wtype: int, w: np.ndarray, rows: int, cols: int, mode: str) -> tp.TpProjection:
        shard = tp.shard_weight(wtype, w, rows, cols, mode, self.rank, self.world)
        buf = self.be.import_host_readonly(shard.weights.reshape(-1))
        variant = 0
        if wtype in (synth.Q6_K, synth.Q8_0, synth.Q4_0) and shard.cols % 256 == 0 and shard.rows > 0:
            # what a loader does once per weight: the repacked row layout of the tensor-core kernel for these types
            st = hb.Stream(self.be, self.stream())
            packed = self.be.repack(st, wtype, hb.TensorRef.of(buf), shard.rows, shard.cols)
            torch.cuda.current_stream(self.device).synchronize()
            buf.free()
            buf, variant = packed, capi.GEMV_MMA_R
        self._weights[id(shard)] = buf
        shard.weights = np.empty((0, 0), np.uint8)  # the host copy is not needed any more
        return tp.TpProjection(shard, lambda s, x, _b=buf, _v=variant: self.matmul(s, _b, x, _v),
                               self.all_reduce if mode == "row" else None)

    def matmul(self, s: tp.Shard, wbuf: hb.Buffer, x: torch.Tensor, variant: int = 0) -> torch.Tensor:
        x = x.contiguous()
        n_vec = x.shape[0]
        y = torch.empty((n_vec, s.rows), dtype=torch.float32, device=self.device)
        g = capi.Gemv()
        g.wtype, g.variant_id = s.wtype, variant
        g.w, g.w_stride = wbuf.ptr, 0
        g.x, g.x_stride = x.data_ptr(), x.stride(0) * 4
        g.y, g.y_stride = y.data_ptr(), 0
        g.rows, g.cols, g.n_vec, g.flags = s.rows, s.cols, n_vec, 0
        rc = self.be.lib.halo_cuda_gemv(self.be.ctx, C.byref(g), self.stream())
        if rc != 0:
            raise hb.HaloError(rc, capi.last_error())
        return y

    def all_reduce(self, y: torch.Tensor) -> None:
        if self.world > 1:
            dist.all_reduce(y)
