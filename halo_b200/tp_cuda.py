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
from . import capi, gguf, synth, tp


def variant_pushes(wtype: int, variant: int) -> bool:
    """Whether the kernel a projection runs has the peer epilogue: the tensor-core skinny variants."""
    return variant in capi.REPACKED_VARIANTS or (variant == 0 and wtype == synth.Q4_K)


class CudaTp:
    def __init__(self, device: int, rank: int, world: int):
        self.be = hb.CudaBackend(device)
        self.rank, self.world = rank, world
        self.device = torch.device("cuda", device)
        self._weights: dict[int, hb.Buffer] = {}
        self.peers: capi.PeerReduce | None = None
        self._peer_bufs: list[hb.Buffer] = []
        self._peer_maps: list[int] = []

    def enable_peer_reduce(self, capacity: int) -> None:
        """Sets up the peer-memory all-reduce epilogue of the row-split projections: a receive buffer of 2 x world slots of
        `capacity` 8-byte words per rank, exchanged as IPC handles over torch.distributed."""
        if self.world == 1 or self.peers is not None:
            return
        lib, ctx = self.be.lib, self.be.ctx
        slots = self.be.allocate(2 * self.world * capacity * 8, shareable=True)
        words = self.be.allocate(64)
        self._peer_bufs = [slots, words]
        torch.cuda.synchronize(self.device)
        h = C.create_string_buffer(64)
        rc = lib.halo_cuda_ipc_export(ctx, C.c_void_p(slots.ptr), h)
        if rc != 0:
            raise hb.HaloError(rc, capi.last_error())
        mine = bytes(h.raw)
        everyone: list = [None] * self.world
        dist.all_gather_object(everyone, mine)
        pr = capi.PeerReduce()
        pr.world, pr.rank, pr.capacity = self.world, self.rank, capacity
        for p, handle in enumerate(everyone):
            if p == self.rank:
                pr.slots[p] = slots.ptr
                continue
            out = C.c_void_p()
            rc = lib.halo_cuda_ipc_open(ctx, handle, C.byref(out))
            if rc != 0:
                raise hb.HaloError(rc, capi.last_error())
            pr.slots[p] = out.value
            self._peer_maps.append(out.value)
        pr.epoch, pr.done = words.ptr, words.ptr + 16
        self.peers = pr
        dist.barrier()  # nobody pushes before every rank has mapped its peers

    def close(self) -> None:
        if self.peers is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier()  # no peer may still be writing into a buffer that is about to go
            for ptr in self._peer_maps:
                self.be.lib.halo_cuda_ipc_close(self.be.ctx, C.c_void_p(ptr))
            self.peers, self._peer_maps = None, []

    def stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def load(self, wtype: int, w: np.ndarray, rows: int, cols: int, mode: str) -> tp.TpProjection:
        shard = tp.shard_weight(wtype, w, rows, cols, mode, self.rank, self.world)
        buf = self.be.import_host_readonly(shard.weights.reshape(-1))
        variant = 0
        if tp.repacks(wtype, rows, cols, mode, self.world) and shard.rows > 0:
            # what a loader does once per weight: the repacked row layout of the tensor-core kernel for these types
            st = hb.Stream(self.be, self.stream())
            packed = self.be.repack(st, wtype, hb.TensorRef.of(buf), shard.rows, shard.cols)
            torch.cuda.current_stream(self.device).synchronize()
            buf.free()
            buf, variant = packed, self.be.repacked_variant(wtype, tp.largest_local_cols(wtype, cols, mode, self.world))
        shard.weights = np.empty((0, 0), np.uint8)  # the host copy is not needed any more
        return self._projection(shard, buf, variant)

    def load_group(self, wtype: int, members: list[tuple[np.ndarray, int]], cols: int) -> tuple[tp.TpProjection, list[tuple[int, int]]]:
        """Projections that share one x, loaded as one column-split operand (one launch per rank instead of one per member);
        returns the projection and each member's (offset, rows) inside this rank's y."""
        shard, where = tp.shard_group(wtype, members, cols, self.rank, self.world)
        buf = self.be.import_host_readonly(shard.weights.reshape(-1)) if shard.rows else self.be.allocate(16)
        variant = 0
        if tp.repacks(wtype, shard.rows, cols, "column", self.world) and shard.rows > 0:
            st = hb.Stream(self.be, self.stream())
            packed = self.be.repack(st, wtype, hb.TensorRef.of(buf), shard.rows, shard.cols)
            torch.cuda.current_stream(self.device).synchronize()
            buf.free()
            buf, variant = packed, self.be.repacked_variant(wtype, cols)
        shard.weights = np.empty((0, 0), np.uint8)
        return self._projection(shard, buf, variant), where

    def load_file(self, f: gguf.GgufFile, info: gguf.TensorInfo, mode: str) -> tp.TpProjection:
        """The same projection straight from a GGUF file: the loader cuts this rank's share out of the mapping, stages it through
        pinned memory and repacks it on the device where the kernels have a repacked layout."""
        split = {"column": capi.SPLIT_COLUMN, "row": capi.SPLIT_ROW}[mode]
        m = gguf.upload_matrix(self.be, hb.Stream(self.be, self.stream()), f, info, split, self.rank, self.world, repack=True)
        torch.cuda.current_stream(self.device).synchronize()
        shard = tp.Shard(mode, self.rank, self.world, m.wtype, m.rows, m.cols, m.row0, m.k0, np.empty((0, 0), np.uint8))
        return self._projection(shard, m.buf if m.buf is not None else self.be.allocate(16), m.variant_id)

    def _projection(self, shard: tp.Shard, buf: hb.Buffer, variant: int) -> tp.TpProjection:
        mode, wtype = shard.mode, shard.wtype
        self._weights[id(shard)] = buf
        if mode == "row" and self.peers is not None and variant_pushes(wtype, variant):
            # the matmul kernel pushes its rows to the peers and a small kernel adds them: no separate collective
            p = tp.TpProjection(shard, lambda s, x, _b=buf, _v=variant: self.matmul(s, _b, x, _v, reduce=True), None, fused=True)
        else:
            p = tp.TpProjection(shard, lambda s, x, _b=buf, _v=variant: self.matmul(s, _b, x, _v), self.all_reduce if mode == "row" else None)
        p.buf, p.variant = buf, variant  # what a caller needs to build the same projection with another reduction
        return p

    def matmul(self, s: tp.Shard, wbuf: hb.Buffer, x: torch.Tensor, variant: int = 0, reduce: bool = False) -> torch.Tensor:
        x = x.contiguous()
        n_vec = x.shape[0]
        y = torch.empty((n_vec, s.rows), dtype=torch.float32, device=self.device)
        g = capi.Gemv()
        g.wtype, g.variant_id = s.wtype, variant
        g.w, g.w_stride = wbuf.ptr, 0
        g.x, g.x_stride = x.data_ptr(), x.stride(0) * 4
        g.y, g.y_stride = y.data_ptr(), 0
        g.rows, g.cols, g.n_vec, g.flags = s.rows, s.cols, n_vec, 0
        if reduce:
            rc = self.be.lib.halo_cuda_gemv_reduce(self.be.ctx, C.byref(g), C.byref(self.peers), self.stream())
        else:
            rc = self.be.lib.halo_cuda_gemv(self.be.ctx, C.byref(g), self.stream())
        if rc != 0:
            raise hb.HaloError(rc, capi.last_error())
        return y

    def all_reduce(self, y: torch.Tensor) -> None:
        if self.world > 1:
            dist.all_reduce(y)
