"""Shared fixtures.  Tests marked `gpu` need a B200; everything else runs on CPU."""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle_c():
    import oracle
    return oracle.Oracle()


@pytest.fixture(scope="session")
def checker():
    """The compiled reference when it travelled with the tree, else the C restatement."""
    import oracle
    return oracle.best_checker()


def sha256(a: np.ndarray) -> bytes:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest()


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def golden(name: str):
    return np.load(GOLDEN / name)
