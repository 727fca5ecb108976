"""The allocation-free entry point (gtk_encode_chunks_noalloc) against the regular
device-resident entry point, through the C ABI.  Collected last on purpose.

Some users of the library tokenise from places where device memory may not be allocated any
more -- a serving loop with a frozen memory budget, or a process whose framework allocator already
owns all of HBM.  For them the library carries one kernel variant whose working memory is a fixed
array inside the library image.  This test checks that the variant produces the same ids as the
regular path and as the CPU oracle, twice in a row (the array keeps the previous call's contents),
that it honours the handle's id space, that a chunk bound beyond the fixed array's capacity is
refused with a clear message, and that chunk offsets pointing outside the text come back as an
error code with the offending chunks skipped (the kernel never uses them as indices).
"""
from __future__ import annotations

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _unpack(ids_at_offsets: np.ndarray, counts: np.ndarray, chunk_off: np.ndarray) -> np.ndarray:
    return np.concatenate([ids_at_offsets[s:s + n] for s, n in zip(chunk_off[:-1], counts)] or [np.zeros(0, np.int32)])


def test_no_alloc_entry_point_matches_regular_path(native_built, merges_path, oracle):
    import torch
    from oracle.loader import MODE_SEGMENTED

    import gputok_b200
    from gputok_b200.capi import NOALLOC_MAX_CHUNK_BYTES

    rng = np.random.default_rng(5)
    # chunk lengths on both sides of the shared-memory limit (8192) so the fixed workspace is used,
    # plus empty, tiny and maximum-size chunks; stress text so long repeated runs occur
    lens = np.concatenate([rng.integers(1, 3000, size=300), rng.integers(8193, NOALLOC_MAX_CHUNK_BYTES, size=40),
                           [0, 1, 2, NOALLOC_MAX_CHUNK_BYTES, 8192, 8193, 0]])
    rng.shuffle(lens)
    chunk_off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    n = int(chunk_off[-1])
    data = gputok_b200.TextGen(6).text(n, mix=gputok_b200.MIX_STRESS)
    data[:NOALLOC_MAX_CHUNK_BYTES] = ord("a")            # one long run across the first chunks

    tok = gputok_b200.Tokenizer(merges_path, chunk_tokens=NOALLOC_MAX_CHUNK_BYTES, device=0)
    # torch fills the buffers below on its current stream: run the library on that stream too
    tok.set_stream(torch.cuda.current_stream().cuda_stream)
    d_bytes = torch.from_numpy(data.copy()).cuda()
    d_off = torch.from_numpy(chunk_off).cuda()
    n_chunks = len(lens)

    # regular entry point: every "text" is one chunk, packed output
    d_ids = torch.empty(n, dtype=torch.int32, device="cuda")
    d_coff = torch.empty(n_chunks + 8, dtype=torch.int64, device="cuda")
    n_ids, n_c, _ = tok.encode_device(d_bytes.data_ptr(), n, d_off.data_ptr(), n_chunks, d_ids.data_ptr(), n,
                                      d_coff.data_ptr(), d_coff.numel())
    want = d_ids[:n_ids].cpu().numpy()
    want_counts = np.diff(d_coff[:n_c + 1].cpu().numpy())
    nonempty = lens > 0
    assert n_c == int(nonempty.sum())
    # the CPU oracle on exactly these chunks (Algorithm 1 per never-merge segment: the 16 KiB chunks would
    # take the literal quadratic loop seconds each; test_oracle.py proves the two equal)
    o_ids, o_off = oracle.encode_chunks(data, chunk_off, mode=MODE_SEGMENTED, threads=8)
    assert np.array_equal(want, o_ids), "regular entry point differs from the oracle"

    for call in range(2):                                 # two calls in a row share the fixed array
        out_ids = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        out_cnt = torch.full((n_chunks,), -1, dtype=torch.int32, device="cuda")
        tok.encode_chunks_noalloc(d_bytes.data_ptr(), n, d_off.data_ptr(), n_chunks, NOALLOC_MAX_CHUNK_BYTES,
                                  out_ids.data_ptr(), out_cnt.data_ptr())
        counts = out_cnt.cpu().numpy()
        assert np.array_equal(counts[nonempty], want_counts), f"call {call}: per-chunk counts differ"
        assert (counts[~nonempty] == 0).all()
        got = _unpack(out_ids.cpu().numpy(), counts, chunk_off)
        assert np.array_equal(got, want), f"call {call}: ids differ from the regular entry point"
        assert np.array_equal(got, o_ids) and np.array_equal(counts, np.diff(o_off)), f"call {call}: differs from the oracle"

    with pytest.raises(gputok_b200.GtkError) as e:        # beyond the fixed array: refused up front
        tok.encode_chunks_noalloc(d_bytes.data_ptr(), n, d_off.data_ptr(), n_chunks, NOALLOC_MAX_CHUNK_BYTES + 1,
                                  out_ids.data_ptr(), out_cnt.data_ptr())
    assert e.value.code == 4 and "exceeds the allocation-free limit" in str(e.value)
    with pytest.raises(gputok_b200.GtkError) as e:        # a chunk that breaks the caller's own bound
        tok.encode_chunks_noalloc(d_bytes.data_ptr(), n, d_off.data_ptr(), n_chunks, 4096, out_ids.data_ptr(),
                                  out_cnt.data_ptr())
    assert e.value.code == 4


    # GPT-2 id space: ids below 256 are remapped exactly as the regular entry point remaps them
    tok.set_id_space(True)
    n_ids2, _, _ = tok.encode_device(d_bytes.data_ptr(), n, d_off.data_ptr(), n_chunks, d_ids.data_ptr(), n,
                                     d_coff.data_ptr(), d_coff.numel())
    want2 = d_ids[:n_ids2].cpu().numpy()
    assert n_ids2 == n_ids and not np.array_equal(want2, want)
    tok.encode_chunks_noalloc(d_bytes.data_ptr(), n, d_off.data_ptr(), n_chunks, NOALLOC_MAX_CHUNK_BYTES,
                              out_ids.data_ptr(), out_cnt.data_ptr())
    got2 = _unpack(out_ids.cpu().numpy(), out_cnt.cpu().numpy(), chunk_off)
    assert np.array_equal(got2, want2), "GPT-2 id space: ids differ from the regular entry point"
    tok.set_id_space(False)

    # offsets that leave the text: error code, offending chunks skipped, the others still tokenised
    bad = chunk_off.copy()
    bad[-1] = n + 4096                                    # last chunk runs past n_bytes
    bad_neg = chunk_off.copy()
    bad_neg[0] = -64                                      # first chunk starts before the text
    for arr, skipped in ((bad, n_chunks - 1), (bad_neg, 0)):
        d_bad = torch.from_numpy(arr).cuda()
        out_ids.fill_(-1)
        out_cnt.fill_(-1)
        with pytest.raises(gputok_b200.GtkError) as e:
            tok.encode_chunks_noalloc(d_bytes.data_ptr(), n, d_bad.data_ptr(), n_chunks, NOALLOC_MAX_CHUNK_BYTES,
                                      out_ids.data_ptr(), out_cnt.data_ptr())
        assert e.value.code == 1 and "inside [0, n_bytes]" in str(e.value)
        counts = out_cnt.cpu().numpy()
        assert counts[skipped] == 0
        keep = np.ones(n_chunks, bool)
        keep[skipped] = False
        assert np.array_equal(counts[keep], np.diff(o_off)[keep])
