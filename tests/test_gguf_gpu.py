"""GGUF file -> device operand (halo_cuda_upload_matrix): the bytes that arrive are the bytes of the file (whole matrix, column
share, row share; several staging turns), a repacking upload equals repacking after a plain import, and the matmul over an
uploaded operand is bitwise the matmul over the same weights imported directly."""
from __future__ import annotations

import numpy as np
import pytest

import gguf_image as gi
from conftest import bits
from halo_b200 import backend as hb
from halo_b200 import capi, synth, tp
from halo_b200.gguf import GgufFile, upload_matrix

pytestmark = pytest.mark.gpu
F32 = 0
SHAPES = {synth.Q4_K: (70, 2560), synth.Q6_K: (37, 3072), synth.Q8_0: (50, 1536), synth.Q4_0: (129, 2048)}


@pytest.fixture(scope="module")
def be():
    return hb.CudaBackend(0)


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    tensors, raws = [], {}
    for i, (t, (rows, cols)) in enumerate(SHAPES.items()):
        w = synth.quant_weights(t, rows, cols, seed=0, tensor_id=10 + i)
        raws[t] = np.ascontiguousarray(w).view(np.uint8).reshape(rows, -1)
        tensors.append((f"blk.{i}.ffn_up.weight", [cols, rows], t, raws[t].tobytes()))
    dense = synth.normal_f32(0, 30, (9, 160))
    raws[F32] = dense.view(np.uint8).reshape(9, -1)
    tensors.append(("dense.weight", [160, 9], F32, dense.tobytes()))
    tensors.append(("norm.weight", [64], F32, bytes(256)))
    tensors.append(("blk.9.q5.weight", [256, 4], 13, bytes(4 * 176)))
    tensors.append(("cube.weight", [32, 2, 3], synth.Q8_0, bytes(6 * 34)))
    infos, data = gi.place(tensors)
    path = tmp_path_factory.mktemp("gguf") / "model.gguf"
    path.write_bytes(gi.image([gi.kv("general.architecture", gi.STRING, "qwen35")], infos, data))
    return GgufFile.open(path), raws


def fetch(be, st, m) -> np.ndarray:
    out = np.empty(m.rows * m.row_stride, np.uint8)
    if out.size:
        be.download(st, hb.TensorRef.of(m.buf), out)
    st.wait()
    return out.reshape(m.rows, -1) if m.rows else out


@pytest.mark.parametrize("t", list(SHAPES) + [F32])
def test_uploaded_bytes_are_the_file_bytes(be, model, t):
    f, raws = model
    st = be.create_stream()
    info = [x for x in f.tensors() if x.type == t and x.n_dims == 2 and x.name != "blk.9.q5.weight"][0]
    rows, cols = info.ne[1], info.ne[0]
    # a whole matrix in one turn, and in many turns of a few rows each
    for staging in (0, 3 * raws[t].shape[1] + 5, 1):
        m = upload_matrix(be, st, f, info, staging_bytes=staging)
        assert (m.rows, m.cols, m.row0, m.k0, m.variant_id, m.wtype) == (rows, cols, 0, 0, 0, t)
        assert np.array_equal(fetch(be, st, m), raws[t])
    if t == F32:
        return
    for world in (2, 3, 8):
        for rank in range(world):
            for mode, split in (("column", capi.SPLIT_COLUMN), ("row", capi.SPLIT_ROW)):
                want = tp.shard_weight(t, raws[t], rows, cols, mode, rank, world)
                m = upload_matrix(be, st, f, info, split, rank, world, staging_bytes=4096)
                assert (m.rows, m.cols, m.row0, m.k0) == (want.rows, want.cols, want.row0, want.k0), (mode, rank, world)
                got = fetch(be, st, m)
                assert got.size == want.weights.size and np.array_equal(got.reshape(-1), want.weights.reshape(-1)), (mode, rank, world)


@pytest.mark.parametrize("t", [synth.Q6_K, synth.Q8_0, synth.Q4_0])
def test_repacking_upload_equals_repack_after_import(be, model, t):
    f, raws = model
    st = be.create_stream()
    info = [x for x in f.tensors() if x.type == t and x.n_dims == 2][0]
    rows, cols = info.ne[1], info.ne[0]
    for split, rank, world in ((capi.SPLIT_NONE, 0, 1), (capi.SPLIT_COLUMN, 1, 3), (capi.SPLIT_ROW, 0, 2), (capi.SPLIT_ROW, 7, 8)):
        m = upload_matrix(be, st, f, info, split, rank, world, repack=True, staging_bytes=8192)
        mode = {capi.SPLIT_NONE: "column", capi.SPLIT_COLUMN: "column", capi.SPLIT_ROW: "row"}[split]
        want = tp.shard_weight(t, raws[t], rows, cols, mode, rank, world)
        if want.cols % 256 != 0:
            assert m.variant_id == capi.GEMV_DEFAULT and np.array_equal(fetch(be, st, m).reshape(-1), want.weights.reshape(-1))
            continue
        assert m.variant_id == capi.GEMV_MMA_I8X2_R and m.row_stride == be.repacked_row_bytes(t, want.cols)
        wb = be.import_host_readonly(want.weights.reshape(-1))
        pk = be.repack(st, t, hb.TensorRef.of(wb), want.rows, want.cols)
        ref = np.empty(want.rows * m.row_stride, np.uint8)
        be.download(st, hb.TensorRef.of(pk), ref)
        st.wait()
        assert np.array_equal(fetch(be, st, m).reshape(-1), ref)


@pytest.mark.parametrize("t", list(SHAPES))
@pytest.mark.parametrize("n_vec", [1, 5])
def test_matmul_over_an_uploaded_operand(be, model, checker, t, n_vec):
    """Bitwise the product over directly imported weights, and -- with the exact-order variant -- bitwise the CPU backend's."""
    f, raws = model
    st = be.create_stream()
    info = [x for x in f.tensors() if x.type == t and x.n_dims == 2][0]
    rows, cols = info.ne[1], info.ne[0]
    x = synth.activations(n_vec, cols, seed=3)
    xb = be.import_host_readonly(x)

    def product(wref, variant, r=rows):
        yb = be.allocate(n_vec * r * 4)
        be.gemv(st, hb.GemvArgs(t, wref, hb.TensorRef.of(xb), hb.TensorRef.of(yb), r, cols, n_vec, variant))
        y = np.empty((n_vec, r), np.float32)
        be.download(st, hb.TensorRef.of(yb), y)
        st.wait()
        return y

    m = upload_matrix(be, st, f, info, staging_bytes=10000)
    direct = be.import_host_readonly(raws[t].reshape(-1))
    want = checker.gemv(t, raws[t], x, rows, cols)
    assert np.array_equal(bits(product(m.ref(), capi.GEMV_EXACT8)), bits(want))
    assert np.array_equal(bits(product(m.ref(), 0)), bits(product(hb.TensorRef.of(direct), 0)))
    if t != synth.Q4_K and cols % 256 == 0:
        r = upload_matrix(be, st, f, info, repack=True)
        y = product(r.ref(), r.variant_id)
        assert np.max(np.abs(y - want)) <= 1e-3 * np.max(np.abs(want))
    # a column share gives the corresponding entries of the whole product: bit for bit in the exact-order variant; the balanced
    # kernels may cut K differently for another row count, so the default is held to the summation bound
    share = upload_matrix(be, st, f, info, capi.SPLIT_COLUMN, 1, 3)
    part = want[:, share.row0:share.row0 + share.rows]
    assert np.array_equal(bits(product(share.ref(), capi.GEMV_EXACT8, share.rows)), bits(part))
    # (Q4_K: the default is the int8 family, which rounds x to 16 bits per super-block)
    assert np.max(np.abs(product(share.ref(), 0, share.rows) - part)) <= (2e-4 if t == synth.Q4_K else 1e-5) * np.max(np.abs(want))


def test_upload_refusals(be, model):
    f, _ = model
    st = be.create_stream()
    for name, status in (("blk.9.q5.weight", capi.E_UNSUPPORTED), ("cube.weight", capi.E_MODEL)):
        with pytest.raises(hb.HaloError) as e:
            upload_matrix(be, st, f, f.find_tensor(name))
        assert e.value.status == status
    info = f.find_tensor("blk.0.ffn_up.weight")
    with pytest.raises(hb.HaloError) as e:
        upload_matrix(be, st, f, info, capi.SPLIT_ROW, 4, 4)
    assert e.value.status == capi.E_API
    # a vector is a one-row matrix
    v = upload_matrix(be, st, f, f.find_tensor("norm.weight"))
    assert (v.rows, v.cols) == (1, 64)
    # more ranks than rows: the last ranks hold nothing
    tiny = upload_matrix(be, st, f, f.find_tensor("dense.weight"), capi.SPLIT_COLUMN, 15, 16)
    assert tiny.rows == 0 and tiny.buf is None


@pytest.mark.parametrize("t", list(SHAPES))
def test_tensor_parallel_shares_loaded_from_the_file(model, t):
    """Every rank's projection loaded by the tensor-parallel harness from the file (the ranks run one after another on this
    device): column shares are the rows of the whole product and row shares add up to it, both within the summation bound."""
    import torch
    from halo_b200 import tp_cuda
    f, raws = model
    info = [x for x in f.tensors() if x.type == t and x.n_dims == 2][0]
    rows, cols = info.ne[1], info.ne[0]
    x = torch.from_numpy(synth.activations(3, cols, seed=5)).cuda()
    whole_tp = tp_cuda.CudaTp(0, 0, 1)
    whole = whole_tp.load_file(f, info, "column")
    y = whole.matmul(whole.shard, x).cpu().numpy()
    for world in (2, 4):
        parts, total = [], np.zeros_like(y, dtype=np.float64)
        for rank in range(world):
            g = tp_cuda.CudaTp(0, rank, world)
            col = g.load_file(f, info, "column")
            parts.append(col.matmul(col.shard, x).cpu().numpy())
            row = g.load_file(f, info, "row")
            total += row.matmul(row.shard, row.local_x(x)).cpu().numpy()
        got = np.concatenate(parts, axis=1)
        assert np.max(np.abs(got - y)) <= 1e-5 * np.max(np.abs(y))
        assert np.max(np.abs(total - y)) <= 1e-4 * np.max(np.abs(y))
