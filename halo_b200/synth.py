"""Seeded synthetic GGUF-layout weights and activations.

There is no model file on the test or benchmark machines, so every tensor is drawn from a
counter-based SplitMix64 stream keyed by (seed, tensor id): element i of a tensor depends on
nothing but the key and i, which makes any slice reproducible on its own.  The block fields
follow the layouts of the reference's dequantizers (src/tensor/quant.cpp:79-90, 143-151,
247-269, 302-327): quants and sub-block codes are uniform over their whole code range and the
fp16 super-block scales are uniform on [0.001, 0.02].
"""
from __future__ import annotations

import numpy as np

F32, Q4_0, Q8_0, Q4_K, Q6_K = 0, 2, 8, 12, 14
TYPE_NAMES = {F32: "f32", Q4_0: "q4_0", Q8_0: "q8_0", Q4_K: "q4_k", Q6_K: "q6_k"}
TYPE_IDS = {v: k for k, v in TYPE_NAMES.items()}
BLOCK_ELEMS = {F32: 1, Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {F32: 4, Q4_0: 18, Q8_0: 34, Q4_K: 144, Q6_K: 210}
# byte offsets of the fp16 scale fields inside one block
_SCALE_FIELDS = {Q4_0: (0,), Q8_0: (0,), Q4_K: (0, 2), Q6_K: (208,)}

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def row_bytes(wtype: int, cols: int) -> int:
    """Bytes of one weight row of `cols` elements (src/tensor/quant.cpp:422-428)."""
    be = BLOCK_ELEMS[wtype]
    if cols % be != 0:
        raise ValueError(f"{cols} elements is not a multiple of the {TYPE_NAMES[wtype]} block size {be}")
    return cols // be * BLOCK_BYTES[wtype]


def _mix(z: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = z + _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def stream_u64(seed: int, tensor_id: int, n: int, start: int = 0) -> np.ndarray:
    """n 64-bit draws, numbers start .. start+n-1 of the stream keyed by (seed, tensor_id)."""
    with np.errstate(over="ignore"):
        key = _mix(np.array([np.uint64(seed) * _M1 + np.uint64(tensor_id)], np.uint64))[0]
        idx = np.arange(start, start + n, dtype=np.uint64)
        return _mix(key + idx * _GOLDEN)


def uniform01(z: np.ndarray) -> np.ndarray:
    """Top 53 bits as a double in [0, 1)."""
    return (z >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def normal_f32(seed: int, tensor_id: int, shape) -> np.ndarray:
    """fp32 ~ N(0, 1) by Box-Muller on two uniforms per element."""
    n = int(np.prod(shape))
    z = stream_u64(seed, tensor_id, 2 * n)
    u1 = (uniform01(z[0::2]) + 1.0 / 9007199254740992.0)  # (0, 1]
    u2 = uniform01(z[1::2])
    v = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return v.astype(np.float32).reshape(shape)


def random_bytes(seed: int, tensor_id: int, n: int) -> np.ndarray:
    return stream_u64(seed, tensor_id, (n + 7) // 8).view(np.uint8)[:n].copy()


def quant_weights(wtype: int, rows: int, cols: int, seed: int = 0, tensor_id: int = 1, *, d_lo: float = 0.001,
                  d_hi: float = 0.02) -> np.ndarray:
    """`rows` dense rows of `cols` elements in the GGUF layout of `wtype`, as uint8 [rows, row_bytes]."""
    if wtype == F32:
        return normal_f32(seed, tensor_id, (rows, cols)).view(np.uint8).reshape(rows, cols * 4)
    rb = row_bytes(wtype, cols)
    nblk = rows * (cols // BLOCK_ELEMS[wtype])
    bb = BLOCK_BYTES[wtype]
    raw = random_bytes(seed, tensor_id, nblk * bb).reshape(nblk, bb)
    if wtype == Q8_0:
        q = raw[:, 2:].view(np.int8)
        q[q == -128] = -127  # quants uniform on [-127, 127]
    if wtype == Q6_K:
        s = raw[:, 192:208]
        s[:] = (s.astype(np.int32) % 128 - 64).astype(np.int8).view(np.uint8)  # sub-block scales on [-64, 63]
    for k, off in enumerate(_SCALE_FIELDS[wtype]):
        u = uniform01(stream_u64(seed, tensor_id + 0x10000 * (k + 1), nblk))
        d = (d_lo + (d_hi - d_lo) * u).astype(np.float32).astype(np.float16)  # round to nearest even
        raw[:, off:off + 2] = d.view(np.uint8).reshape(nblk, 2)
    return raw.reshape(rows, rb)


def random_blocks_finite(wtype: int, rows: int, cols: int, seed: int, tensor_id: int = 1) -> np.ndarray:
    """Fully random block bytes with every fp16 scale forced finite: 2^U(-12, 2) with a random sign
    (the recipe of the reference's synthetic dequant fixture, python/tools/fetch_quant_blocks.py:219-236)."""
    rb = row_bytes(wtype, cols)
    nblk = rows * (cols // BLOCK_ELEMS[wtype])
    bb = BLOCK_BYTES[wtype]
    raw = random_bytes(seed, tensor_id, nblk * bb).reshape(nblk, bb)
    for k, off in enumerate(_SCALE_FIELDS[wtype]):
        z = stream_u64(seed, tensor_id + 0x10000 * (k + 1), nblk)
        mag = np.exp2(-12.0 + 14.0 * uniform01(z))
        sign = np.where((z & np.uint64(1)) == 0, 1.0, -1.0)
        d = (mag * sign).astype(np.float32).astype(np.float16)
        raw[:, off:off + 2] = d.view(np.uint8).reshape(nblk, 2)
    return raw.reshape(rows, rb)


def activations(n_vec: int, cols: int, seed: int = 0, tensor_id: int = 2) -> np.ndarray:
    return normal_f32(seed, tensor_id, (n_vec, cols))
