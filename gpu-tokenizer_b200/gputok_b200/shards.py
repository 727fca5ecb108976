"""Byte-range sharding of a batch over GPUs and stitching of the results.

Chunks are independent, so a batch is cut into contiguous runs of texts, one
run per GPU, balanced by bytes; every GPU tokenises its run on its own and the
only cross-GPU step is adding the running id count to each shard's offsets on
the host.  No collective touches the data path.
"""
from __future__ import annotations

import numpy as np


def partition_by_bytes(text_offsets, n_shards: int) -> np.ndarray:
    """Split texts 0..T into n_shards contiguous runs with near-equal byte counts.

    Returns int64[n_shards+1] text indices: shard s owns texts bounds[s]..bounds[s+1].
    A text is never split (its chunks stay on one GPU).
    """
    off = np.asarray(text_offsets, dtype=np.int64)
    n_texts = len(off) - 1
    total = int(off[-1] - off[0]) if n_texts > 0 else 0
    bounds = np.zeros(n_shards + 1, dtype=np.int64)
    for s in range(1, n_shards):
        target = off[0] + (total * s) // n_shards
        # first text boundary at or after the target byte
        t = int(np.searchsorted(off, target, side="left"))
        bounds[s] = min(max(t, bounds[s - 1]), n_texts)
    bounds[n_shards] = n_texts
    return bounds


def split_single_text(n_bytes: int, chunk_bytes: int, n_shards: int) -> np.ndarray:
    """Byte ranges for one long text cut at chunk boundaries (so the shards' chunking
    equals the chunking of the whole).  Returns int64[n_shards+1] byte offsets."""
    n_chunks = (n_bytes + chunk_bytes - 1) // chunk_bytes
    bounds = np.zeros(n_shards + 1, dtype=np.int64)
    for s in range(1, n_shards + 1):
        bounds[s] = min(((n_chunks * s) // n_shards) * chunk_bytes, n_bytes)
    bounds[n_shards] = n_bytes
    return bounds


def stitch_offsets(shard_offsets: list[np.ndarray]) -> np.ndarray:
    """Concatenate per-shard id offsets (each starting at 0) into global offsets."""
    out = [np.zeros(1, dtype=np.int64)]
    base = 0
    for off in shard_offsets:
        off = np.asarray(off, dtype=np.int64)
        out.append(off[1:] + base)
        base += int(off[-1])
    return np.concatenate(out)


def imbalance(values) -> float:
    """max / mean of per-shard work or time (1.0 = perfectly balanced)."""
    v = np.asarray(values, dtype=np.float64)
    return float(v.max() / v.mean()) if len(v) and v.mean() > 0 else 1.0
