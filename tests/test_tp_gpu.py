"""Tensor-parallel projections on real GPUs: launched by pytest as torchrun children when at least two devices are
present; every rank checks its results against the single-GPU result of the same projection."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu

CHILD = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["HALO_ROOT"])
from halo_b200 import synth, tp, tp_cuda, capi
rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(lr)
dist.init_process_group("nccl", device_id=torch.device("cuda", lr))
rt = tp_cuda.CudaTp(lr, rank, world)
one = tp_cuda.CudaTp(lr, 0, 1)   # the single-GPU oracle on the same device
for wtype, rows, cols, m in [(synth.Q4_K, 1024, 5120, 1), (synth.Q6_K, 512, 4352, 4), (synth.Q4_K, 640, 6144, 3)]:
    w = synth.quant_weights(wtype, rows, cols, 31, 1)
    x = torch.from_numpy(synth.activations(m, cols, 31, 2)).cuda()
    full = one.load(wtype, w, rows, cols, "column")(x)
    col = rt.load(wtype, w, rows, cols, "column")
    y = col(x)
    n0 = col.shard.row0
    assert torch.equal(y.view(torch.int32), full[:, n0:n0 + col.shard.rows].contiguous().view(torch.int32)), "column split must be bitwise"
    row = rt.load(wtype, w, rows, cols, "row")
    yr = row(x)
    err = (yr - full).abs().max().item() / full.abs().max().item()
    assert err <= 1e-5, f"row split + all-reduce off by {err}"
    ref = yr.clone(); dist.broadcast(ref, 0)
    assert torch.equal(ref.view(torch.int32), yr.view(torch.int32)), "every rank must hold the same reduced y"
# the same row splits with the peer-memory epilogue: the matmul kernel pushes its rows to the peers, a small kernel adds them
rt.enable_peer_reduce(16 * 1024)
for wtype, rows, cols, m in [(synth.Q4_K, 1024, 5120, 1), (synth.Q6_K, 512, 4352, 4), (synth.Q4_K, 640, 6144, 3), (synth.Q4_K, 37, 1024, 16), (synth.Q4_K, 200, 2048, 21)]:
    w = synth.quant_weights(wtype, rows, cols, 33, 1)
    x = torch.from_numpy(synth.activations(m, cols, 33, 2)).cuda()
    full = one.load(wtype, w, rows, cols, "column")(x)
    rt.peers, keep = None, rt.peers
    nccl = rt.load(wtype, w, rows, cols, "row")(x)       # partial products + NCCL all-reduce
    rt.peers = keep
    fused = rt.load(wtype, w, rows, cols, "row")
    assert fused.fused and fused.all_reduce is None, "the fused projection must not call a collective"
    for it in range(5):                                     # both ping-pong slot sets, several times over
        yf = fused(x)
        err = (yf - full).abs().max().item() / full.abs().max().item()
        assert err <= 1e-5, f"peer-reduced row split off by {err} (iteration {it})"
        if world == 2:                                      # two addends: the order cannot matter
            assert torch.equal(yf.view(torch.int32), nccl.view(torch.int32)), "peer reduction differs from the NCCL all-reduce"
        ref = yf.clone(); dist.broadcast(ref, 0)
        assert torch.equal(ref.view(torch.int32), yf.view(torch.int32)), "every rank must hold the same reduced y"
st = rt.be.create_stream(); st.wait()                      # raises if a flag wait expired on the device
rt.close()
torch.cuda.synchronize(); dist.barrier(); dist.destroy_process_group()
print("TP_OK", rank)
'''


def test_tp_two_ranks_nccl(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, HALO_ROOT=str(ROOT), NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29731", str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.count("TP_OK") == 2, r.stdout[-2000:] + r.stderr[-3000:]
