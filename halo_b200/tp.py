"""Tensor-parallel weight split for the matmul path: one process per GPU, torch.distributed for the plumbing.

The reference has no multi-GPU code; the single-GPU result of the same projection is the oracle for every split.

* Column split (QKV / gate / up, and the vocabulary of the LM head): each rank keeps whole W rows
  [n0, n1); x is replicated; no communication.  A rank's outputs are bitwise the corresponding entries of the
  single-GPU result, because a row's arithmetic never looks at other rows.
* Row split (o / out / down): each rank keeps the K range [k0, k1) of every row, cut at whole quantization blocks
  (256 elements for Q4_K / Q6_K, 32 for Q8_0 / Q4_0).  Where K / tp is not a whole number of blocks the shares are
  uneven (K = 5120 over 8 ranks: 3,3,3,3,2,2,2,2 super-blocks).  Each rank computes a full-length partial y from its
  slice of x, and the partials are summed by an all-reduce.  The sum is split differently from the single-GPU one:
  parity is bounded, not bitwise.
* LM head: a column split whose per-rank argmax triples carry the rank's row offset; merging them by "larger value,
  then lower index" gives the single-GPU winner because that order is total (backends/cpu/matmul.cpp:19-22).

The arithmetic is injected (`matmul`, `all_reduce`): the GPU path passes the cuda backend and NCCL, the CPU tests
pass a checker and gloo.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import numpy as np

from .synth import BLOCK_BYTES, BLOCK_ELEMS, row_bytes


def split_even(n: int, parts: int) -> list[tuple[int, int]]:
    """[begin, end) of each part when n items go to `parts` contiguous parts; the first n % parts get one more
    (the reference's static partition, include/halo/backends/cpu/thread_pool.h:64-72)."""
    base, extra = divmod(n, parts)
    out, b = [], 0
    for i in range(parts):
        e = b + base + (1 if i < extra else 0)
        out.append((b, e))
        b = e
    return out


def column_ranges(rows: int, tp: int) -> list[tuple[int, int]]:
    """W rows of each rank."""
    return split_even(rows, tp)


def row_ranges(wtype: int, cols: int, tp: int) -> list[tuple[int, int]]:
    """K range (in elements) of each rank, cut at whole blocks of `wtype`."""
    be = BLOCK_ELEMS[wtype]
    if cols % be != 0:
        raise ValueError(f"{cols} columns is not a whole number of {be}-element blocks")
    return [(b * be, e * be) for b, e in split_even(cols // be, tp)]


def repacks(wtype: int, rows: int, cols: int, mode: str, tp: int) -> bool:
    """Whether the ranks of a split keep their shares in the repacked row layout of the tensor-core kernels (Q6_K / Q8_0 / Q4_0,
    whole 256-element groups).  The layout selects the kernel variant and with it how a row split is reduced (peer epilogue or
    collective), so the answer is a function of the GLOBAL shape: every rank computes the same one.  A row split repacks only
    when every rank's K share is a non-empty whole number of groups."""
    from .synth import Q4_0, Q6_K, Q8_0
    if wtype not in (Q6_K, Q8_0, Q4_0) or rows == 0 or cols == 0:
        return False
    if mode == "row":
        return all(e > b and (e - b) % 256 == 0 for b, e in row_ranges(wtype, cols, tp))
    return cols % 256 == 0


def largest_local_cols(wtype: int, cols: int, mode: str, tp: int) -> int:
    """The largest K any rank multiplies: what decides the kernel variant of a repacked tensor, alike on every rank."""
    if mode != "row":
        return cols
    return max(e - b for b, e in row_ranges(wtype, cols, tp))


@dataclass
class Shard:
    mode: str            # "column" | "row"
    rank: int
    tp: int
    wtype: int
    rows: int            # local W rows
    cols: int            # local K
    row0: int            # first global row (column split) or 0
    k0: int              # first global K element (row split) or 0
    weights: np.ndarray  # dense local rows, uint8 [rows, row_bytes(wtype, cols)]


def shard_weight(wtype: int, w: np.ndarray, rows: int, cols: int, mode: str, rank: int, tp: int) -> Shard:
    """The local part of a dense quantized matrix `w` (uint8 [rows, row_bytes]) for `rank` of `tp`."""
    rb = row_bytes(wtype, cols)
    w = np.ascontiguousarray(w).view(np.uint8).reshape(rows, rb)
    if mode == "column":
        n0, n1 = column_ranges(rows, tp)[rank]
        return Shard(mode, rank, tp, wtype, n1 - n0, cols, n0, 0, np.ascontiguousarray(w[n0:n1]))
    if mode == "row":
        k0, k1 = row_ranges(wtype, cols, tp)[rank]
        be, bb = BLOCK_ELEMS[wtype], BLOCK_BYTES[wtype]
        return Shard(mode, rank, tp, wtype, rows, k1 - k0, 0, k0, np.ascontiguousarray(w[:, k0 // be * bb:k1 // be * bb]))
    raise ValueError(f"unknown split mode {mode!r}")


def shard_group(wtype: int, members: list[tuple[np.ndarray, int]], cols: int, rank: int, tp: int) -> tuple[Shard, list[tuple[int, int]]]:
    """Several projections that read the same x (the reference's fused qkv, beta|alpha and gate|up operands,
    src/models/qwen35.cpp:79-96, 220-253) as ONE column-split operand: every member is split over the ranks on its own and a
    rank's rows are its member shares back to back, so that one matmul per rank produces its slice of every member.
    `members`: (dense rows as uint8 [rows, row_bytes], rows).  Returns the shard and, per member, (offset, rows) of its
    slice inside the rank's y."""
    parts, where, at = [], [], 0
    for w, rows in members:
        s = shard_weight(wtype, w, rows, cols, "column", rank, tp)
        parts.append(s.weights)
        where.append((at, s.rows))
        at += s.rows
    rb = row_bytes(wtype, cols)
    weights = np.concatenate(parts, axis=0) if at else np.empty((0, rb), np.uint8)
    return Shard("column", rank, tp, wtype, at, cols, 0, 0, weights), where


class TpProjection:
    """y = x W^T over a tensor-parallel group.

    matmul(shard, x_local) -> y_partial  runs the local product ([n_vec, shard.cols] -> [n_vec, shard.rows]);
    all_reduce(y)                       sums y in place over the group (row split only).
    """

    def __init__(self, shard: Shard, matmul: Callable, all_reduce: Callable | None = None, fused: bool = False):
        """fused: `matmul` already returns the sum over the group (a kernel with a reduction epilogue)."""
        if shard.mode == "row" and shard.tp > 1 and all_reduce is None and not fused:
            raise ValueError("a row split needs an all-reduce")
        self.shard, self.matmul, self.all_reduce, self.fused = shard, matmul, all_reduce, fused

    def local_x(self, x):
        """The slice of a full-width x this rank multiplies (row split), or x itself (column split)."""
        s = self.shard
        if s.mode != "row" or x.shape[-1] == s.cols:
            return x  # column split, or the caller already holds only its K range (the output of a column split)
        return x[..., s.k0:s.k0 + s.cols]

    def __call__(self, x):
        s = self.shard
        y = self.matmul(s, self.local_x(x))
        if s.mode == "row" and s.tp > 1 and not self.fused:
            self.all_reduce(y)
        return y


def merge_argmax(triples: list[np.ndarray]) -> np.ndarray:
    """Per-rank LM-head result words {index (already offset), value bits, nan} -> the group's winner per vector.
    A vector poisoned on any rank stays poisoned: {0xFFFFFFFF, quiet NaN, 1}."""
    stack = np.stack([np.ascontiguousarray(t, np.uint32).reshape(-1, 3) for t in triples])  # [tp, n_vec, 3]
    n_vec = stack.shape[1]
    out = np.zeros((n_vec, 3), np.uint32)
    for v in range(n_vec):
        if np.any(stack[:, v, 2] != 0):
            out[v] = (0xFFFFFFFF, 0x7FC00000, 1)
            continue
        best = None
        for r in range(stack.shape[0]):
            idx, bits = int(stack[r, v, 0]), stack[r, v, 1]
            if idx == 0xFFFFFFFF:
                continue
            val = float(np.array([bits], np.uint32).view(np.float32)[0])
            if best is None or val > best[0] or (val == best[0] and idx < best[1]):
                best = (val, idx, bits)
        out[v] = (0xFFFFFFFF, 0, 0) if best is None else (best[1], best[2], 0)
    return out
