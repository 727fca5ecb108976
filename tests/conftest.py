"""Shared fixtures.  Tests marked ``gpu`` need a B200 and call the CUDA library through its
C ABI; everything else runs on CPU (oracle, host logic, symbol checks, gloo sharding)."""
from __future__ import annotations

import gzip
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "gpu-tokenizer_b200")
GOLDEN = os.path.join(ROOT, "tests", "golden")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

MERGES = os.path.join(GOLDEN, "gpt2_merges.txt")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def merges_path() -> str:
    return MERGES


@pytest.fixture(scope="session")
def native_built():
    """Build the native libraries once (nvcc cross-compiles without a GPU)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("gtk_build", os.path.join(PKG, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build_all()
    return mod


@pytest.fixture(scope="session")
def oracle(merges_path):
    from oracle.loader import Oracle, build

    build(ref=os.path.isdir("/root/reference"))
    return Oracle(merges_path)


@pytest.fixture(scope="session")
def novel() -> bytes:
    with gzip.open(os.path.join(GOLDEN, "pride_and_prejudice.txt.gz"), "rb") as f:
        return f.read()


@pytest.fixture(scope="session")
def golden_2048():
    z = np.load(os.path.join(GOLDEN, "golden_blockbpe_2048.npz"))
    return z["ids"].astype(np.int32), z["offsets"].astype(np.int64)


@pytest.fixture(scope="session")
def ref_cases():
    return dict(np.load(os.path.join(GOLDEN, "ref_greedy_cases.npz")))


def fixed_chunk_offsets(n: int, chunk: int) -> np.ndarray:
    off = list(range(0, n, chunk)) + [n]
    return np.array(off if n else [0], dtype=np.int64)


def first_mismatch(a: np.ndarray, b: np.ndarray) -> str:
    n = min(len(a), len(b))
    d = np.flatnonzero(a[:n] != b[:n])
    if len(d):
        i = int(d[0])
        return f"first difference at {i}: {a[max(0, i - 4):i + 6].tolist()} vs {b[max(0, i - 4):i + 6].tolist()}"
    return f"lengths {len(a)} vs {len(b)}"
