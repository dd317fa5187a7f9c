"""Builds libhalo_cuda_backend.so: the C++23 `halo::backend::Backend` implementation over the C ABI.

It compiles against the reference's own headers where they lie ($HALO_REF_ROOT, else a directory `reference` next to this repository); nothing of the
reference is copied.  Without the reference tree (e.g. on the GPU box) the prebuilt library that travelled with the
tree is used as is.  Symbols of HALO's backend-neutral code (op_name, Backend::run_op, ...) stay undefined in this
library: the HALO build, or the test that loads it, provides them.
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
PKG = HERE.parent
LIB = HERE / "libhalo_cuda_backend.so"


def ref_root() -> Path | None:
    env = os.environ.get("HALO_REF_ROOT")
    for root in ([Path(env)] if env else []) + [PKG.parent.parent / "reference"]:
        if (root / "include" / "halo" / "backend" / "backend.h").exists():
            return root
    return None


def build(force: bool = False) -> Path | None:
    root = ref_root()
    if root is None:
        return LIB if LIB.exists() else None
    srcs = [HERE / "cuda_backend.cpp"]
    deps = srcs + [HERE / "cuda_backend.h", PKG.parent / "include" / "halo_cuda.h", PKG / "libhalo_cuda.so"]
    if not force and LIB.exists() and all(LIB.stat().st_mtime >= d.stat().st_mtime for d in deps if d.exists()):
        return LIB
    cmd = ["g++", "-std=c++23", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-Wall", "-Wextra", f"-I{root / 'include'}",
           f"-I{PKG.parent / 'include'}", *map(str, srcs), "-o", str(LIB), f"-L{PKG}", "-l:libhalo_cuda.so", "-Wl,-rpath,$ORIGIN/.."]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
