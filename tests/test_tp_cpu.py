"""Host logic of the tensor-parallel split on CPU: partitions, shard extraction, and a world_size-2 gloo run in which
the local products come from the checker.  The single-rank result is the oracle for every split."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest

from conftest import bits
from halo_b200 import synth, tp

ROOT = Path(__file__).resolve().parents[1]


def test_partitions():
    assert tp.column_ranges(17408, 8) == [(i * 2176, (i + 1) * 2176) for i in range(8)]
    # K = 5120 is 20 super-blocks: 8 ranks get 3,3,3,3,2,2,2,2
    r = tp.row_ranges(synth.Q4_K, 5120, 8)
    assert [(e - b) // 256 for b, e in r] == [3, 3, 3, 3, 2, 2, 2, 2] and r[0][0] == 0 and r[-1][1] == 5120
    # K = 17408 is 68 super-blocks: 9,9,9,9,8,8,8,8
    assert [(e - b) // 256 for b, e in tp.row_ranges(synth.Q6_K, 17408, 8)] == [9, 9, 9, 9, 8, 8, 8, 8]
    assert tp.row_ranges(synth.Q8_0, 17408, 4) == [(i * 4352, (i + 1) * 4352) for i in range(4)]
    with pytest.raises(ValueError):
        tp.row_ranges(synth.Q4_K, 1000, 2)
    assert tp.column_ranges(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]


@pytest.mark.parametrize("wtype", [synth.Q4_K, synth.Q6_K, synth.Q8_0, synth.Q4_0])
def test_shards_reassemble_and_match_the_single_rank_result(oracle_c, wtype):
    rows, cols, m, n_ranks = 48, 2048, 3, 3
    w = synth.quant_weights(wtype, rows, cols, 21, 1)
    x = synth.activations(m, cols, 21, 2)
    full = oracle_c.gemv(wtype, w, x, rows, cols)

    def matmul(s, xl):
        return oracle_c.gemv(s.wtype, s.weights, np.ascontiguousarray(xl), s.rows, s.cols)

    # column split: concatenated rank outputs are bitwise the single-rank result
    parts = [tp.TpProjection(tp.shard_weight(wtype, w, rows, cols, "column", r, n_ranks), matmul)(x) for r in range(n_ranks)]
    assert np.array_equal(bits(np.concatenate(parts, axis=1)), bits(full))
    # row split: shard bytes are exactly the block ranges, and the summed partials agree within the summation bound
    shards = [tp.shard_weight(wtype, w, rows, cols, "row", r, n_ranks) for r in range(n_ranks)]
    assert sum(s.cols for s in shards) == cols
    assert np.array_equal(np.concatenate([s.weights for s in shards], axis=1), w)
    acc = np.zeros_like(full)
    for s in shards:
        acc += tp.TpProjection(s, matmul, all_reduce=lambda y: None)(x)
    wf = oracle_c.dequantize(wtype, w, rows * cols).reshape(rows, cols).astype(np.float64)
    bound = 2 * (cols // 8 + 8) * 2.0**-24 * (np.abs(x.astype(np.float64)) @ np.abs(wf).T)
    assert np.all(np.abs(acc.astype(np.float64) - full) <= bound)


def test_merge_argmax_is_the_single_call_answer(oracle_c):
    V, E, n, ranks = 4096, 256, 4, 4
    w = synth.quant_weights(synth.Q8_0, V, E, 22, 1)
    x = synth.activations(n, E, 22, 2)
    x[2, 0] = np.nan
    full, _, _ = oracle_c.lm_head(synth.Q8_0, w, x, V, E, want_logits=False)
    triples = []
    for r in range(ranks):
        s = tp.shard_weight(synth.Q8_0, w, V, E, "column", r, ranks)
        res, _, _ = oracle_c.lm_head(synth.Q8_0, s.weights, x, s.rows, E, want_logits=False)
        res = res.copy()
        ok = res[:, 0] != 0xFFFFFFFF
        res[ok, 0] += s.row0  # what halo_cuda_lm_head does with row_offset
        triples.append(res)
    assert np.array_equal(tp.merge_argmax(triples), full)


def _worker(rank: int, world: int, port: int, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    import oracle
    dist.init_process_group("gloo", rank=rank, world_size=world)
    chk = oracle.Oracle()
    rows, cols, m = 40, 2560, 2
    w = synth.quant_weights(synth.Q4_K, rows, cols, 23, 1)
    x = synth.activations(m, cols, 23, 2)

    def matmul(s, xl):
        return torch.from_numpy(chk.gemv(s.wtype, s.weights, np.ascontiguousarray(xl), s.rows, s.cols, threads=1))

    up = tp.TpProjection(tp.shard_weight(synth.Q4_K, w, rows, cols, "column", rank, world), matmul)
    down = tp.TpProjection(tp.shard_weight(synth.Q4_K, w, rows, cols, "row", rank, world), matmul, all_reduce=lambda y: dist.all_reduce(y))
    y_col = up(x)
    gathered = [torch.zeros_like(y_col) for _ in range(world)]
    dist.all_gather(gathered, y_col)
    y_row = down(x)
    q.put((rank, torch.cat(gathered, dim=1).numpy(), y_row.numpy()))
    dist.barrier()
    dist.destroy_process_group()


def _file_worker(rank: int, world: int, port: int, path: str, q):
    """Each rank cuts its own shares out of the GGUF file with the loader's share arithmetic (no device needed)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    import torch
    import torch.distributed as dist

    import oracle
    from halo_b200 import capi, gguf
    dist.init_process_group("gloo", rank=rank, world_size=world)
    chk = oracle.Oracle()
    f = gguf.GgufFile.open(path)
    out = {}
    for info in f.tensors():
        rows, cols = info.ne[1], info.ne[0]
        x = synth.activations(2, cols, 31, 2)
        mc, wc = gguf.host_share(f, info, capi.SPLIT_COLUMN, rank, world)
        y_col = torch.from_numpy(chk.gemv(info.type, np.ascontiguousarray(wc), x, mc.rows, cols, threads=1))
        sizes = [gguf.matrix_share(info.type, rows, cols, capi.SPLIT_COLUMN, r, world).rows for r in range(world)]
        gathered = [torch.zeros((2, n), dtype=torch.float32) for n in sizes]
        gathered[rank] = y_col
        for r in range(world):  # shares may differ in size (41 rows over 2 ranks), so every rank broadcasts its own
            dist.broadcast(gathered[r], r)
        mr, wr = gguf.host_share(f, info, capi.SPLIT_ROW, rank, world)
        y_row = torch.from_numpy(chk.gemv(info.type, np.ascontiguousarray(wr), np.ascontiguousarray(x[:, mr.k0:mr.k0 + mr.cols]), rows, mr.cols, threads=1))
        dist.all_reduce(y_row)
        out[info.name] = (torch.cat(gathered, dim=1).numpy(), y_row.numpy())
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_load_their_shares_from_a_gguf_file(oracle_c, tmp_path):
    import torch.multiprocessing as mp

    from halo_b200 import gguf
    shapes = {"blk.0.ffn_up.weight": (synth.Q4_K, 41, 1280), "blk.0.ffn_down.weight": (synth.Q6_K, 24, 1792), "blk.0.attn_q.weight": (synth.Q8_0, 30, 416),
              "output.weight": (synth.Q4_0, 17, 800)}
    raws = {n: synth.quant_weights(t, r, c, 31, 1 + i) for i, (n, (t, r, c)) in enumerate(shapes.items())}
    path = tmp_path / "tp.gguf"
    gguf.write_gguf(path, [(n, t, r, c, raws[n]) for n, (t, r, c) in shapes.items()], {"general.architecture": "qwen35"})
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_file_worker, args=(r, 2, port, str(path), q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for name, (t, rows, cols) in shapes.items():
        full = oracle_c.gemv(t, raws[name], synth.activations(2, cols, 31, 2), rows, cols)
        for _, out in results:
            y_col, y_row = out[name]
            assert np.array_equal(bits(y_col), bits(full)), name                       # column shares: bitwise
            assert np.max(np.abs(y_row - full)) <= 1e-5 * np.max(np.abs(full)), name   # row shares + all-reduce: bounded


def test_two_gloo_ranks_column_and_row_split(oracle_c):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    rows, cols, m = 40, 2560, 2
    w = synth.quant_weights(synth.Q4_K, rows, cols, 23, 1)
    x = synth.activations(m, cols, 23, 2)
    full = oracle_c.gemv(synth.Q4_K, w, x, rows, cols)
    for _, y_col, y_row in results:
        assert np.array_equal(bits(y_col), bits(full))                       # column split: bitwise
        assert np.max(np.abs(y_row - full)) <= 1e-5 * np.max(np.abs(full))   # row split + all-reduce: bounded
    assert np.array_equal(bits(results[0][2]), bits(results[1][2]))          # every rank holds the same reduced y


def test_every_rank_of_a_split_chooses_the_same_kernel_layout():
    """The repacked layout selects the kernel variant, and the variant selects how a row split is reduced (peer epilogue or
    collective): ranks that disagreed would wait for each other in different protocols.  With blocks of 32 elements the K
    shares can be uneven across ranks (K = 544 over two ranks: 288 and 256 columns), so the decision must come from the
    global shape -- in the Python split and in the loader of the C ABI alike."""
    from halo_b200 import capi, gguf
    cases = [(synth.Q8_0, 40, 544, 2), (synth.Q4_0, 40, 544, 2), (synth.Q8_0, 40, 1536, 4), (synth.Q8_0, 40, 1536, 2), (synth.Q6_K, 40, 5120, 8),
             (synth.Q4_0, 40, 768, 3), (synth.Q8_0, 40, 17408, 4), (synth.Q6_K, 3, 512, 4), (synth.Q4_K, 40, 5120, 8)]
    for wtype, rows, cols, world in cases:
        for mode, split in (("row", capi.SPLIT_ROW), ("column", capi.SPLIT_COLUMN)):
            want = tp.repacks(wtype, rows, cols, mode, world)
            variants = set()
            for rank in range(world):
                m = gguf.matrix_share(wtype, rows, cols, split, rank, world, repack=True)
                if m.rows and m.cols:  # a rank without rows holds nothing and launches nothing
                    variants.add(m.variant_id)
            assert len(variants) <= 1, (wtype, rows, cols, world, mode)
            if variants:
                assert (variants <= set(capi.REPACKED_VARIANTS)) == want, (wtype, rows, cols, world, mode)
    assert not tp.repacks(synth.Q8_0, 40, 544, "row", 2)       # 288 + 256 columns: one rank could repack, the other not
    assert tp.repacks(synth.Q8_0, 40, 1536, "row", 2) and not tp.repacks(synth.Q8_0, 40, 1536, "row", 4)
    assert tp.repacks(synth.Q6_K, 40, 5120, "row", 8)           # 3,3,3,3,2,2,2,2 super-blocks: all whole groups


def test_grouped_projections_are_the_members_side_by_side(oracle_c):
    """qkv | z | beta | alpha as one operand: every rank's y holds its column share of each member, bitwise what the member's own
    projection gives (a row's arithmetic never looks at other rows in the CPU order)."""
    cols, m, ranks = 1024, 2, 3
    sizes = [80, 48, 6, 6]
    ws = [synth.quant_weights(synth.Q4_K, n, cols, 41, i + 1) for i, n in enumerate(sizes)]
    x = synth.activations(m, cols, 41, 9)

    def matmul(s, xl):
        return oracle_c.gemv(s.wtype, s.weights, np.ascontiguousarray(xl), s.rows, s.cols)

    for r in range(ranks):
        shard, where = tp.shard_group(synth.Q4_K, list(zip(ws, sizes)), cols, r, ranks)
        assert shard.rows == sum(n for _, n in where)
        y = tp.TpProjection(shard, matmul)(x)
        for (at, n), w, rows in zip(where, ws, sizes):
            own = tp.TpProjection(tp.shard_weight(synth.Q4_K, w, rows, cols, "column", r, ranks), matmul)(x)
            assert own.shape[1] == n and np.array_equal(bits(y[:, at:at + n]), bits(own))
