"""Generates the committed golden vectors from the reference itself.

Run in a container that has the reference tree (so that oracle/_ref/libhalo_ref.so can be
built) and gguf-py 0.19.0 (the dequantizer the reference's own zero-tolerance test cites,
tests/unit/tensor/test_quant_blocks.cpp:1-8):

    python tests/golden/make_golden.py

Outputs (all under tests/golden/):
  dequant.npz   block bytes -> fp32, produced by the reference's tensor::dequantize_row AND by
                gguf.quants.dequantize (the script refuses to write if the two disagree)
  gemv.npz      Backend::gemv outputs of the reference CPU backend for small odd shapes
  lm_head.npz   Backend::lm_head result triples / logits across the 8192-row slab boundary
  fp16.npz      fp16 -> fp32 for all 65536 inputs, fp32 -> fp16 for a seeded sample + edge cases
Weights larger than a few KB are stored as a generator recipe plus a SHA-256 of the bytes.
"""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from halo_b200 import synth  # noqa: E402

OUT = Path(__file__).resolve().parent
TYPES = (synth.Q4_0, synth.Q8_0, synth.Q4_K, synth.Q6_K)


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    import gguf
    from gguf import quants

    oracle.build()
    ref = oracle.Reference()
    gq = {synth.Q4_0: gguf.GGMLQuantizationType.Q4_0, synth.Q8_0: gguf.GGMLQuantizationType.Q8_0,
          synth.Q4_K: gguf.GGMLQuantizationType.Q4_K, synth.Q6_K: gguf.GGMLQuantizationType.Q6_K}

    # ---- dequant: the reference's synthetic fixture recipe (seed 20260923, 2 rows, 8 blocks) -------------
    d = {}
    for t in TYPES:
        cols = 8 * synth.BLOCK_ELEMS[t]
        for label, w in (("rand", synth.random_blocks_finite(t, 2, cols, 20260923, t)),
                         ("cfg", synth.quant_weights(t, 2, cols, 0, t))):
            a = ref.dequantize(t, w, 2 * cols)
            g = quants.dequantize(w, gq[t]).astype(np.float32).reshape(-1)
            if not np.array_equal(a.view(np.uint32), g.view(np.uint32)):
                raise SystemExit(f"reference and gguf-py disagree on {synth.TYPE_NAMES[t]} {label}")
            d[f"{synth.TYPE_NAMES[t]}_{label}_bytes"] = w
            d[f"{synth.TYPE_NAMES[t]}_{label}_f32"] = a
    np.savez_compressed(OUT / "dequant.npz", **d)

    # ---- gemv through the reference Backend interface -----------------------------------------------------
    g = {}
    cases = []
    for t in TYPES + (synth.F32,):
        be = synth.BLOCK_ELEMS[t]
        k_small = 512 if be <= 256 else be
        for (n, k, m) in ((37, k_small, 1), (13, 2560, 3), (40, 1024 if t != synth.F32 else 64, 17)):
            cases.append((t, n, k, m))
    for i, (t, n, k, m) in enumerate(cases):
        w = synth.quant_weights(t, n, k, 100 + i, 1)
        x = synth.activations(m, k, 100 + i, 2)
        y = ref.gemv(t, w, x, n, k)
        name = f"c{i}"
        g[name + "_meta"] = np.array([t, n, k, m, 100 + i], np.int64)
        g[name + "_w_sha"] = np.frombuffer(bytes.fromhex(sha(w)), np.uint8)
        g[name + "_x"] = x
        g[name + "_y"] = y
    g["n_cases"] = np.array([len(cases)], np.int64)
    np.savez_compressed(OUT / "gemv.npz", **g)

    # ---- lm_head across the slab boundary, NaN poisoning, valid_rows ----------------------------------------
    h = {}
    V, E, n = 8192 + 900, 256, 3
    for t in (synth.Q8_0, synth.Q4_K):
        w = synth.quant_weights(t, V, E, 200 + t, 1)
        x = synth.activations(n, E, 200 + t, 2)
        res, logits, ids = ref.lm_head(t, w, x, V, E)
        res_v, _, ids_v = ref.lm_head(t, w, x, V, E, valid_rows=5000, want_logits=False)
        x2 = x.copy()
        x2[1, 0] = np.nan
        res_n, _, ids_n = ref.lm_head(t, w, x2, V, E, want_logits=False)
        p = synth.TYPE_NAMES[t]
        h[p + "_meta"] = np.array([t, V, E, n, 200 + t], np.int64)
        h[p + "_w_sha"] = np.frombuffer(bytes.fromhex(sha(w)), np.uint8)
        h[p + "_x"] = x
        h[p + "_result"] = res
        h[p + "_logits"] = logits
        h[p + "_ids"] = ids
        h[p + "_result_valid5000"] = res_v
        h[p + "_ids_valid5000"] = ids_v
        h[p + "_result_nanrow1"] = res_n
        h[p + "_ids_nanrow1"] = ids_n
    np.savez_compressed(OUT / "lm_head.npz", **h)

    # ---- fp16 conversions --------------------------------------------------------------------------------
    widen = np.array([np.float32(ref.fp16_to_fp32(i)) for i in range(65536)], np.float32).view(np.uint32)
    rng_bits = synth.stream_u64(7, 7, 4096).astype(np.uint32)
    edge = np.array([0x00000000, 0x80000000, 0x33000000, 0x33000001, 0x337FFFFF, 0x33800000, 0x387FC000, 0x387FE000,
                     0x38800000, 0x477FE000, 0x477FEFFF, 0x477FF000, 0x47800000, 0x7F800000, 0xFF800000, 0x7FC00000,
                     0x7F800001, 0x3F801000, 0x3F803000, 0x3F801001, 0x3A83126F, 0x3CA3D70A], np.uint32)
    src = np.concatenate([rng_bits, edge])
    narrow = np.array([ref.fp32_to_fp16(float(f)) for f in src.view(np.float32)], np.uint16)
    np.savez_compressed(OUT / "fp16.npz", widen_bits=widen, narrow_src_bits=src, narrow=narrow)
    for f in ("dequant.npz", "gemv.npz", "lm_head.npz", "fp16.npz"):
        print(f, (OUT / f).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
