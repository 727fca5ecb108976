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


def pytest_sessionfinish(session, exitstatus):
    """When the session ran on the bounds-checked build of the library (GPUTOK_B200_LIBRARY points to it),
    report the record of failed index checks; a non-empty record fails the session."""
    import ctypes

    path = os.environ.get("GPUTOK_B200_LIBRARY")
    if not path or not os.path.exists(path):
        return
    lib = ctypes.CDLL(path)
    if not hasattr(lib, "gtk_debug_check_words"):
        return
    words = (ctypes.c_int * 4)()
    rc = lib.gtk_debug_check_words(words, 0, 0)
    print(f"\nCHECKED_BUILD rc={rc} failures={words[3]} first_check={words[0]} value={words[1]} limit={words[2]}")
    if rc != 0 or words[3] != 0:
        session.exitstatus = 3


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

    build()
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


def crowded_bucket_merges(merges_path: str, out_path: str):
    """A merges file whose pair table has a crowded bucket, and text that probes it.

    The device pair table hashes key = left << 16 | right with h = key * 0x9E3779B1 (mod 2**32) into
    bucket h >> 16, four entries per bucket; further keys of a bucket go to a side table.  1024
    first-level merges of byte pairs (ranks 0..1023, ids 256..1279) are followed by second-level
    merges (first-level id, byte) that all fall into the fullest bucket, so at least two of them
    live in the side table.  Returns (text bytes, number of second-level merges).
    """
    from gputok_b200 import Tokenizer

    base = Tokenizer(merges_path, 2048, 50, device=-1)
    sym = [base.token_symbols(b).decode("utf-8") for b in range(256)]
    first = [(a, (a + d) % 256) for d in (3, 50, 101, 200) for a in range(256)]
    assert len(set(first)) == len(first)
    buckets: dict[int, list[tuple[int, int]]] = {}
    for i in range(len(first)):
        for x in range(256):
            key = ((256 + i) << 16) | x
            buckets.setdefault(((key * 0x9E3779B1) & 0xFFFFFFFF) >> 16, []).append((i, x))
    crowd = max(buckets.values(), key=len)
    assert len(crowd) >= 6
    lines = ["#version: 0.2"] + [f"{sym[a]} {sym[b]}" for a, b in first]
    lines += [f"{sym[first[i][0]]}{sym[first[i][1]]} {sym[x]}" for i, x in crowd]
    with open(out_path, "w", encoding="utf-8") as f:
        f.write("\n".join(lines) + "\n")
    rng = np.random.default_rng(5)
    parts = []
    for _ in range(4000):
        i, x = crowd[int(rng.integers(len(crowd)))]
        parts.append(bytes([first[i][0], first[i][1], x]))
        if rng.random() < 0.3:
            parts.append(bytes(rng.integers(0, 256, int(rng.integers(1, 4)), dtype=np.uint8)))
    return b"".join(parts), len(crowd)


def irregular_merges(merges_path: str, out_path: str, n_lines: int = 4000, seed: int = 9) -> None:
    """A merge table without the regularities of GPT-2's file: the first ``n_lines`` merges in shuffled
    order (a merge may outrank the merges that create its parts, and name parts that no earlier line
    produced) with some lines repeated (a repeated pair keeps its first rank but still consumes one, so
    merged ids stop being 256 + rank)."""
    with open(merges_path, encoding="utf-8") as f:
        lines = f.read().split("\n")
    head, body = lines[0], [ln for ln in lines[1:n_lines + 1] if ln]
    rng = np.random.default_rng(seed)
    body = [body[i] for i in rng.permutation(len(body))]
    for at in sorted(rng.integers(10, len(body), 60).tolist(), reverse=True):
        body.insert(at, body[int(rng.integers(0, at))])
    with open(out_path, "w", encoding="utf-8") as f:
        f.write("\n".join([head] + body) + "\n")


def wide_merges(merges_path: str, out_path: str, oracle, text: bytes, extra: int = 16000):
    """A merges file too large for 16-bit ids: GPT-2's 50 000 merges followed by ``extra`` new ones, the most
    frequent adjacent token pairs of ``text`` under the GPT-2 table (so the new, high-ranked merges really
    fire on that text and produce ids above 65 535).  Returns the number of merges written."""
    from collections import Counter

    from oracle.loader import MODE_SEGMENTED

    ids, off = oracle.encode_fixed(text, 1 << 16, mode=MODE_SEGMENTED, threads=os.cpu_count() or 1)
    pairs = Counter()
    for c in range(len(off) - 1):
        a = ids[off[c]:off[c + 1]]
        pairs.update(zip(a[:-1].tolist(), a[1:].tolist()))
    with open(merges_path, encoding="utf-8") as f:
        lines = f.read().split("\n")
    while lines and not lines[-1]:
        lines.pop()
    have = set(lines[1:])
    new = []
    for (l, r), _ in pairs.most_common():
        sl = oracle.token_symbols(l).decode("utf-8")
        sr = oracle.token_symbols(r).decode("utf-8")
        line = f"{sl} {sr}"
        if " " in sl or " " in sr or not sl or not sr or line in have:
            continue
        new.append(line)
        have.add(line)
        if len(new) >= extra:
            break
    lines += new[::-1]  # rarest first: the most frequent pairs get the highest ranks and ids
    with open(out_path, "w", encoding="utf-8") as f:
        f.write("\n".join(lines) + "\n")
    return len(lines) - 1
