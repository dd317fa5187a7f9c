"""Builds tests/native/libadapter_selftest.so: the C++ differential test of the cuda adapter against the reference CPU
backend, both driven through the reference's Backend interface.  Needs the reference headers ($HALO_REF_ROOT, else a directory `reference` next to this repository) and
oracle/_ref/libhalo_ref.so; where they are absent the prebuilt library that travelled with the tree is used."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
LIB = HERE / "libadapter_selftest.so"


def build(force: bool = False) -> Path | None:
    env = os.environ.get("HALO_REF_ROOT")
    ref = Path(env) if env else ROOT.parent / "reference"
    ref_so = ROOT / "oracle" / "_ref" / "libhalo_ref.so"
    adapter = ROOT / "halo_b200" / "adapter" / "libhalo_cuda_backend.so"
    if not (ref / "include" / "halo" / "backend" / "backend.h").exists() or not ref_so.exists() or not adapter.exists():
        return LIB if LIB.exists() else None
    src = HERE / "adapter_selftest.cpp"
    if not force and LIB.exists() and all(LIB.stat().st_mtime >= p.stat().st_mtime for p in (src, ref_so, adapter)):
        return LIB
    cmd = ["g++", "-std=c++23", "-O1", "-ffp-contract=off", "-fPIC", "-shared", "-Wall", f"-I{ref / 'include'}", f"-I{ROOT / 'include'}",
           f"-I{ROOT / 'halo_b200' / 'adapter'}", str(src), "-o", str(LIB), f"-L{adapter.parent}", "-l:libhalo_cuda_backend.so",
           f"-L{ref_so.parent}", "-l:libhalo_ref.so", f"-L{ROOT / 'halo_b200'}", "-l:libhalo_cuda.so",
           "-Wl,-rpath,$ORIGIN/../../halo_b200/adapter:$ORIGIN/../../oracle/_ref:$ORIGIN/../../halo_b200"]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    sys.path.insert(0, str(ROOT))
    print(build(force=True))
