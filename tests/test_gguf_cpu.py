"""The GGUF index of the weight loader (include/halo_cuda_gguf.h) on CPU: against gguf-py on well-formed files, and
against deliberately damaged images.  Mirrors what the reference tests of its parser (tests/unit/model/test_gguf.cpp):
typed metadata, tensor geometry, alignment, and a typed error -- never a crash -- for every malformed field.
"""
from __future__ import annotations

import ctypes as C
import struct

import numpy as np
import pytest

import gguf_image as gi
from halo_b200 import capi, synth, tp
from halo_b200.backend import HaloError
from halo_b200.gguf import GgufFile, matrix_share

Q4_0, Q8_0, Q4_K, Q5_K, Q6_K, F32, F16 = 2, 8, 12, 13, 14, 0, 1


def code_of(exc) -> int:
    return exc.value.status


def small_model(alignment: int = 32):
    tensors = [
        ("blk.0.ffn_up.weight", [512, 6], Q4_K, gi.random_bytes(1, 6 * 2 * 144)),
        ("blk.0.ffn_down.weight", [256, 5], Q6_K, gi.random_bytes(2, 5 * 210)),
        ("blk.0.attn_q.weight", [64, 3], Q8_0, gi.random_bytes(3, 3 * 2 * 34)),
        ("output.weight", [96, 7], Q4_0, gi.random_bytes(4, 7 * 3 * 18)),
        ("blk.0.attn_norm.weight", [10], F32, np.arange(10, dtype=np.float32).tobytes()),
        ("blk.0.ssm_out.weight", [256, 2], Q5_K, gi.random_bytes(5, 2 * 176)),
        ("token_embd.weight", [8, 4], F16, gi.random_bytes(6, 64)),
    ]
    kvs = [gi.kv("general.architecture", gi.STRING, "qwen35"), gi.kv("qwen35.block_count", gi.U32, 64),
           gi.kv("qwen35.attention.layer_norm_rms_epsilon", gi.F32, 1e-6), gi.kv("t.i8", gi.I8, -5), gi.kv("t.u64", gi.U64, 2 ** 63 + 1),
           gi.kv("t.i64", gi.I64, -2 ** 40), gi.kv("t.f64", gi.F64, 0.125), gi.kv("t.bool", gi.BOOL, 1), gi.kv("t.u16", gi.U16, 65535),
           gi.kv("tokenizer.ggml.tokens", gi.ARRAY, (gi.STRING, ["a", "bc", ""])), gi.kv("t.sections", gi.ARRAY, (gi.I32, [11, 11, 10, 0])),
           gi.kv("t.nested", gi.ARRAY, (gi.ARRAY, [(gi.U8, [1, 2]), (gi.U8, [])])), gi.kv("t.bools", gi.ARRAY, (gi.BOOL, [0, 1, 1]))]
    if alignment != 32:
        kvs.append(gi.kv("general.alignment", gi.U32, alignment))
    infos, data = gi.place(tensors, alignment)
    return gi.image(kvs, infos, data, alignment), tensors


def test_own_image_index_and_typed_metadata():
    img, tensors = small_model()
    f = GgufFile.parse(img)
    assert (f.version, f.alignment, f.n_kv, f.n_tensors, f.file_size) == (3, 32, 13, 7, len(img))
    assert f.data_offset % 32 == 0 and f.header_size <= f.data_offset < f.header_size + 32
    assert f.get_string("general.architecture") == "qwen35"
    assert f.get_uint("qwen35.block_count") == 64 and f.get_int("qwen35.block_count") == 64
    assert f.get_float("qwen35.attention.layer_norm_rms_epsilon") == float(np.float32(1e-6))
    assert f.get_int("t.i8") == -5 and f.get_uint("t.u64") == 2 ** 63 + 1 and f.get_int("t.i64") == -2 ** 40
    assert f.get_float("t.f64") == 0.125 and f.get_uint("t.u16") == 65535 and f.get_uint("absent") is None
    assert f.get_string("absent") is None
    # a present key whose type cannot represent the request: Error(Model), as GgufFile::get_uint / get_string
    for bad in (lambda: f.get_uint("t.i8"), lambda: f.get_int("t.u64"), lambda: f.get_uint("general.architecture"),
                lambda: f.get_string("qwen35.block_count"), lambda: f.get_float("qwen35.block_count"), lambda: f.get_uint("t.bool")):
        with pytest.raises(HaloError) as e:
            bad()
        assert code_of(e) == capi.E_MODEL
    for i, (name, ne, type_id, raw) in enumerate(tensors):
        t = f.find_tensor(name)
        assert t.index == i and t.name == name and t.type == type_id and t.n_dims == len(ne)
        assert list(t.ne[:len(ne)]) == ne and all(e == 1 for e in t.ne[len(ne):])
        assert t.n_bytes == len(raw) and t.offset % 32 == 0 and t.supported == (type_id in (Q4_0, Q8_0, Q4_K, Q6_K, F32))
        assert f.tensor_data(t).tobytes() == raw
    assert f.find_tensor("nope") is None
    with pytest.raises(HaloError) as e:
        f.tensor(7)
    assert code_of(e) == capi.E_API


def test_custom_alignment_and_file_mapping(tmp_path):
    img, tensors = small_model(alignment=256)
    p = tmp_path / "m.gguf"
    p.write_bytes(img)
    with GgufFile.open(p) as f:
        assert f.alignment == 256 and f.data_offset % 256 == 0
        for name, _ne, _t, raw in tensors:
            t = f.find_tensor(name)
            assert t.offset % 256 == 0 and f.tensor_data(t).tobytes() == raw
    with pytest.raises(HaloError) as e:
        GgufFile.open(tmp_path / "missing.gguf")
    assert code_of(e) == capi.E_IO
    with pytest.raises(HaloError) as e:
        GgufFile.open(tmp_path)
    assert code_of(e) == capi.E_IO
    (tmp_path / "empty.gguf").write_bytes(b"")
    with pytest.raises(HaloError) as e:
        GgufFile.open(tmp_path / "empty.gguf")
    assert code_of(e) == capi.E_MODEL


def test_against_gguf_py_writer_and_reader(tmp_path):
    """A file written by gguf-py (the reference's own oracle for the container, tests/unit/tensor/test_quant_blocks.cpp:1-8) reads
    back with the same geometry, offsets and bytes through this index as through gguf-py's reader."""
    gguf = pytest.importorskip("gguf")
    path = tmp_path / "w.gguf"
    w = gguf.GGUFWriter(str(path), "qwen35")
    w.add_uint32("qwen35.block_count", 2)
    w.add_float32("qwen35.rope.freq_base", 1e7)
    w.add_string("general.name", "synthetic")
    w.add_array("qwen35.rope.dimension_sections", [11, 11, 10, 0])
    w.add_array("tokenizer.ggml.tokens", ["<a>", "<b>"])
    rng = np.random.default_rng(7)
    mats = {"blk.0.ffn_gate.weight": (Q4_K, 12, 512), "blk.0.ffn_down.weight": (Q6_K, 9, 768), "blk.1.attn_k.weight": (Q8_0, 5, 96),
            "blk.1.attn_o.weight": (Q4_0, 4, 64)}
    raws = {}
    for name, (t, rows, cols) in mats.items():
        raws[name] = synth.quant_weights(t, rows, cols, seed=len(raws))
        w.add_tensor(name, raws[name].reshape(rows, -1), raw_dtype=gguf.GGMLQuantizationType(t))
    w.add_tensor("output_norm.weight", rng.standard_normal(33).astype(np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    theirs = gguf.GGUFReader(str(path))
    f = GgufFile.open(path)
    assert f.alignment == theirs.alignment and f.n_tensors == len(theirs.tensors)
    assert f.get_uint("qwen35.block_count") == 2 and f.get_string("general.name") == "synthetic"
    assert f.get_float("qwen35.rope.freq_base") == float(np.float32(1e7))
    assert f.get_string("general.architecture") == "qwen35"
    for rt in theirs.tensors:
        t = f.find_tensor(rt.name)
        assert t is not None and t.type == int(rt.tensor_type) and t.n_bytes == rt.n_bytes and t.n_elements == rt.n_elements
        assert list(t.ne[:len(rt.shape)]) == [int(e) for e in rt.shape]
        assert f.data_offset + t.offset == rt.data_offset
        assert f.tensor_data(t).tobytes() == np.ascontiguousarray(rt.data).tobytes()
    for name, (t, rows, cols) in mats.items():
        ti = f.find_tensor(name)
        assert (ti.ne[0], ti.ne[1]) == (cols, rows) and f.tensor_data(ti).tobytes() == raws[name].tobytes()


def test_type_geometry_matches_gguf_py():
    gguf = pytest.importorskip("gguf")
    for qt, (elems, nbytes) in gguf.GGML_QUANT_SIZES.items():
        if int(qt) > 30:
            continue  # ids assigned after the table of this loader: refused as invalid, below
        if int(qt) == 9:
            nbytes = 36  # Q8_1 never reaches a file; ggml's block is two fp16 + 32 int8, the size the reference has too (src/tensor/dtype.cpp:26)
        infos, data = gi.place([("t", [elems * 3, 2], int(qt), bytes(nbytes * 6))])
        f = GgufFile.parse(gi.image([], infos, data))
        t = f.tensor(0)
        assert (t.n_bytes, t.n_elements) == (nbytes * 6, elems * 6), qt
    for bad in (4, 5, 31, 1000):
        with pytest.raises(HaloError) as e:
            GgufFile.parse(gi.image([], [gi.tensor_info("t", [256], bad, 0)], bytes(1024)))
        assert code_of(e) == capi.E_MODEL and "invalid type id" in str(e.value)


# ---- damaged images: a typed error for each, and no read outside the image ------------------------------------------

def parse_fails(img: bytes, status: int, needle: str = ""):
    with pytest.raises(HaloError) as e:
        GgufFile.parse(img)
    assert code_of(e) == status, str(e.value)
    assert needle in str(e.value), str(e.value)


def test_header_errors():
    parse_fails(gi.image([], [], magic=b"GGML"), capi.E_MODEL, "bad magic")
    parse_fails(gi.image([], [], version=1), capi.E_UNSUPPORTED, "v1")
    parse_fails(gi.image([], [], version=struct.unpack("<I", struct.pack(">I", 3))[0]), capi.E_UNSUPPORTED, "big-endian")
    parse_fails(gi.image([], [], version=7), capi.E_MODEL, "unknown GGUF version")
    parse_fails(b"GG", capi.E_MODEL, "truncated")
    parse_fails(gi.image([], [], n_kv=1 << 20), capi.E_MODEL, "exceeds limit")
    parse_fails(gi.image([], [], n_kv=1000), capi.E_MODEL, "cannot fit")
    parse_fails(gi.image([], [], n_tensors=1 << 21), capi.E_MODEL, "exceeds limit")
    parse_fails(gi.image([], [], n_tensors=50), capi.E_MODEL, "cannot fit")
    assert GgufFile.parse(gi.image([], [], version=2)).version == 2
    empty = GgufFile.parse(gi.image([], []))
    assert empty.n_tensors == 0 and empty.n_kv == 0


def test_metadata_errors():
    parse_fails(gi.image([gi.kv("a", gi.U32, 1), gi.kv("a", gi.U32, 2)], []), capi.E_MODEL, "duplicate metadata key")
    parse_fails(gi.image([gi.string("k") + struct.pack("<I", 13) + b"\0" * 8], []), capi.E_MODEL, "invalid GGUF value type")
    parse_fails(gi.image([gi.string("k") + struct.pack("<IIQ", gi.ARRAY, 99, 0)], []), capi.E_MODEL, "array elements")
    parse_fails(gi.image([gi.kv("k", gi.BOOL, 2)], []), capi.E_MODEL, "invalid bool")
    parse_fails(gi.image([gi.kv("k", gi.ARRAY, (gi.BOOL, [1, 3]))], []), capi.E_MODEL, "invalid bool")
    parse_fails(gi.image([gi.string("k") + struct.pack("<IQ", gi.STRING, 1 << 30)], []), capi.E_MODEL, "exceeds limit")
    parse_fails(gi.image([gi.string("k") + struct.pack("<IQ", gi.STRING, 100) + b"abc"], []), capi.E_MODEL, "truncated")
    parse_fails(gi.image([gi.string("k") + struct.pack("<IIQ", gi.ARRAY, gi.U64, 1 << 27)], []), capi.E_MODEL, "exceeds limit")
    parse_fails(gi.image([gi.string("k") + struct.pack("<IIQ", gi.ARRAY, gi.U64, 1 << 20)], []), capi.E_MODEL, "cannot fit")
    nested = (gi.U8, [1])
    for _ in range(8):
        nested = (gi.ARRAY, [nested])
    parse_fails(gi.image([gi.kv("deep", gi.ARRAY, nested)], []), capi.E_MODEL, "nesting deeper")
    ok = (gi.U8, [1])
    for _ in range(7):
        ok = (gi.ARRAY, [ok])
    assert GgufFile.parse(gi.image([gi.kv("deep", gi.ARRAY, ok)], [])).n_kv == 1
    for bad_alignment in (0, 3, 48, 1 << 21):
        parse_fails(gi.image([gi.kv("general.alignment", gi.U32, bad_alignment)], []), capi.E_MODEL, "invalid general.alignment")
    parse_fails(gi.image([gi.kv("general.alignment", gi.U64, 64)], []), capi.E_MODEL, "expected UINT32")


def test_tensor_info_errors():
    blk = bytes(144)
    one = lambda info, data=blk: gi.image([], [info], data)
    parse_fails(one(gi.string("t") + struct.pack("<I", 0) + struct.pack("<IQ", Q4_K, 0)), capi.E_MODEL, "dims")
    parse_fails(one(gi.tensor_info("t", [256, 1, 1, 1, 1], Q4_K, 0)), capi.E_MODEL, "dims")
    parse_fails(one(gi.tensor_info("n" * 64, [256], Q4_K, 0)), capi.E_MODEL, "exceeds limit")
    assert GgufFile.parse(one(gi.tensor_info("n" * 63, [256], Q4_K, 0))).tensor(0).name == "n" * 63
    parse_fails(one(gi.tensor_info("t", [100], Q4_K, 0)), capi.E_MODEL, "multiple of the block size")
    parse_fails(one(gi.tensor_info("t", [1 << 40, 1 << 40], F32, 0)), capi.E_MODEL, "element count overflows")
    parse_fails(one(gi.tensor_info("t", [1 << 63], F32, 0)), capi.E_MODEL, "element count overflows")
    parse_fails(one(gi.tensor_info("t", [1 << 62], 28, 0)), capi.E_MODEL, "byte size overflows")  # F64: 2^65 bytes
    parse_fails(one(gi.tensor_info("t", [256], Q4_K, 16)), capi.E_MODEL, "not a multiple of the alignment")
    parse_fails(one(gi.tensor_info("t", [1 << 61], F32, (1 << 64) - 32)), capi.E_MODEL, "")
    parse_fails(one(gi.tensor_info("t", [512], Q4_K, 0)), capi.E_MODEL, "past end of file")
    parse_fails(one(gi.tensor_info("t", [256], Q4_K, 32)), capi.E_MODEL, "past end of file")
    two = [gi.tensor_info("a", [256], Q4_K, 0), gi.tensor_info("a", [256], Q4_K, 160)]
    parse_fails(gi.image([], two, bytes(320)), capi.E_MODEL, "duplicate tensor name")
    two = [gi.tensor_info("b", [256], Q4_K, 128), gi.tensor_info("a", [512], Q4_K, 0)]
    parse_fails(gi.image([], two, bytes(512)), capi.E_MODEL, "overlaps")
    # zero-sized tensors may share an offset; ne[0] == 0 is a whole number of blocks
    z = GgufFile.parse(gi.image([], [gi.tensor_info("z", [0, 5], Q4_K, 0), gi.tensor_info("y", [256], Q4_K, 0)], blk))
    assert z.tensor(0).n_bytes == 0 and z.tensor_data(z.tensor(0)).size == 0
    # header only, tensors declared but no data section at all
    parse_fails(gi.image([], [gi.tensor_info("t", [256], Q4_K, 0)], b"")[:-1], capi.E_MODEL, "past end of file")


def test_every_truncation_and_single_byte_damage_is_a_typed_error():
    """The file is untrusted input: each prefix of a valid image, and each image with one header byte overwritten, either parses or
    fails with Model / Unsupported -- nothing else, and no crash."""
    img, _ = small_model()
    f = GgufFile.parse(img)
    header, total = f.header_size, len(img)
    for cut in list(range(0, header + 40)) + [total - 1]:
        with pytest.raises(HaloError) as e:
            GgufFile.parse(img[:cut])
        assert code_of(e) in (capi.E_MODEL, capi.E_UNSUPPORTED), cut
    rng = np.random.default_rng(11)
    parsed = 0
    for pos in range(header):
        for v in (0x00, 0xFF, int(rng.integers(1, 255))):
            b = bytearray(img)
            b[pos] = v
            try:
                GgufFile.parse(bytes(b)).tensors()
                parsed += 1
            except HaloError as e:
                assert e.status in (capi.E_MODEL, capi.E_UNSUPPORTED), (pos, v, str(e))
    assert parsed > 0


def test_share_extents_match_the_tensor_parallel_split():
    """halo_cuda_matrix_share deals rows and K blocks exactly as the host-side split of the tensor-parallel harness."""
    for wtype, rows, cols in ((Q4_K, 17408, 5120), (Q6_K, 5120, 17408), (Q8_0, 5120, 17408), (Q4_0, 151936, 5120), (Q4_K, 48, 5120), (Q4_0, 3, 96)):
        for world in (1, 2, 3, 4, 8):
            for rank in range(world):
                m = matrix_share(wtype, rows, cols, capi.SPLIT_COLUMN, rank, world)
                n0, n1 = tp.column_ranges(rows, world)[rank]
                assert (m.row0, m.rows, m.k0, m.cols) == (n0, n1 - n0, 0, cols) and m.row_stride == synth.row_bytes(wtype, cols)
                m = matrix_share(wtype, rows, cols, capi.SPLIT_ROW, rank, world)
                k0, k1 = tp.row_ranges(wtype, cols, world)[rank]
                assert (m.row0, m.rows, m.k0, m.cols) == (0, rows, k0, k1 - k0)
                assert m.row_stride == (synth.row_bytes(wtype, k1 - k0) if k1 > k0 else 0)
    whole = matrix_share(Q6_K, 5120, 17408, repack=True)
    assert whole.variant_id == capi.GEMV_MMA_I8X2_R and whole.row_stride == 17408 // 256 * 224  # 68 super-blocks of x fit next to the ring
    assert matrix_share(Q4_K, 64, 512, repack=True).variant_id == capi.GEMV_DEFAULT  # Q4_K has no repacked layout
    assert matrix_share(Q8_0, 64, 96, repack=True).variant_id == capi.GEMV_DEFAULT   # K is not a whole number of 256-element groups
    assert matrix_share(Q8_0, 50, 1536, capi.SPLIT_ROW, 0, 4, repack=True).variant_id == capi.GEMV_DEFAULT  # 384 local columns: one and a half groups
    assert matrix_share(Q8_0, 50, 1536, capi.SPLIT_ROW, 0, 2, repack=True).variant_id == capi.GEMV_MMA_I8X2_R
    # K beyond what the int8 kernels keep resident: the fp16 family's repacked kernel, which streams x; both ranks of an uneven row
    # split decide from the larger share
    assert matrix_share(Q8_0, 8, 65536, repack=True).variant_id == capi.GEMV_MMA_R
    lib = capi.load()
    v = C.c_uint32()

    def variant(t, k):
        assert lib.halo_cuda_repacked_variant(t, k, C.byref(v)) == 0
        return v.value

    first_r = {}  # per type: the smallest K (a multiple of 256) that no longer fits
    for t in (Q8_0, Q6_K, Q4_0):
        k = 256
        while variant(t, k) == capi.GEMV_MMA_I8X2_R:
            k += 256
        first_r[t] = k
        assert all(variant(t, kk) == capi.GEMV_MMA_R for kk in (k, k + 256, 4 * k))  # monotone: once too long, always too long
    assert first_r[Q8_0] < first_r[Q6_K] < first_r[Q4_0]  # 5 KB, 3.5 KB and 3 KB ring slots leave less, more, most room for x
    assert first_r[Q8_0] > 17408  # every K of the benchmark shapes runs the int8 family
    k_hi, k_lo = first_r[Q6_K], first_r[Q6_K] - 256  # an uneven split into (k_hi, k_lo): rank 1 alone would fit, rank 0 does not
    pair = {matrix_share(Q6_K, 8, k_hi + k_lo, capi.SPLIT_ROW, r, 2, repack=True).variant_id for r in (0, 1)}
    assert pair == {capi.GEMV_MMA_R}
    assert lib.halo_cuda_repacked_variant(Q4_K, 5120, C.byref(v)) == capi.E_UNSUPPORTED
    for bad, status in (((Q5_K, 4, 256), capi.E_UNSUPPORTED), ((Q4_K, 4, 100), capi.E_MODEL)):
        with pytest.raises(HaloError) as e:
            matrix_share(*bad)
        assert code_of(e) == status
    with pytest.raises(HaloError) as e:
        matrix_share(Q4_K, 4, 256, capi.SPLIT_ROW, 2, 2)
    assert code_of(e) == capi.E_API


def test_writer_round_trip(tmp_path):
    """halo_b200.gguf.write_gguf produces a container both this index and gguf-py read back."""
    from halo_b200.gguf import write_gguf
    w = synth.quant_weights(Q6_K, 5, 512, seed=1)
    v = synth.quant_weights(Q4_K, 3, 256, seed=2)
    path = tmp_path / "s.gguf"
    write_gguf(path, [("a.weight", Q6_K, 5, 512, w), ("b.weight", Q4_K, 3, 256, v)], {"general.architecture": "qwen35", "n": 3, "eps": 1.5}, alignment=64)
    f = GgufFile.open(path)
    assert f.alignment == 64 and f.get_uint("n") == 3 and f.get_float("eps") == 1.5 and f.get_string("general.architecture") == "qwen35"
    a, b = f.find_tensor("a.weight"), f.find_tensor("b.weight")
    assert (a.ne[0], a.ne[1], b.ne[0], b.ne[1]) == (512, 5, 256, 3) and a.offset % 64 == 0 and b.offset % 64 == 0
    assert f.tensor_data(a).tobytes() == np.ascontiguousarray(w).tobytes() and f.tensor_data(b).tobytes() == np.ascontiguousarray(v).tobytes()
    gguf = pytest.importorskip("gguf")
    theirs = {t.name: t for t in gguf.GGUFReader(str(path)).tensors}
    assert np.ascontiguousarray(theirs["a.weight"].data).tobytes() == np.ascontiguousarray(w).tobytes()
    assert int(theirs["b.weight"].tensor_type) == Q4_K and theirs["b.weight"].data_offset == f.data_offset + b.offset
