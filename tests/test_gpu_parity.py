"""Parity of the CUDA path with the oracle, through the C ABI, on a B200.

Every comparison is bit-exact (integer ids and offsets).  Small inputs are checked against the
literal Algorithm 1 oracle, full-size configurations against the segmented oracle on every chunk,
the literal oracle on a seeded sample of chunks, and the decode round trip.
"""
from __future__ import annotations

import os

import numpy as np
import pytest

from conftest import first_mismatch, fixed_chunk_offsets, wide_merges
from oracle.loader import MODE_GREEDY, MODE_SEGMENTED

pytestmark = pytest.mark.gpu

NCPU = os.cpu_count() or 1


@pytest.fixture(scope="module")
def lib(native_built):
    import gputok_b200

    # fail loudly if the CUDA library is absent: nothing else can serve these tests
    assert os.path.exists(gputok_b200.library_path())
    return gputok_b200


def make_tok(lib, merges_path, chunk):
    return lib.Tokenizer(merges_path, chunk, 50, device=0)


def check_chunks(ids, coff, want, woff, what):
    assert len(coff) == len(woff), f"{what}: {len(coff) - 1} chunks vs {len(woff) - 1}"
    if not np.array_equal(coff, woff):
        c = int(np.flatnonzero(coff != woff)[0]) - 1
        a, b = ids[coff[c]:coff[c + 1]], want[woff[c]:woff[c + 1]]
        raise AssertionError(f"{what}: chunk {c} differs: {first_mismatch(a, b)}")
    assert np.array_equal(ids, want), f"{what}: {first_mismatch(ids, want)}"


@pytest.mark.parametrize("mode", ["opt", "base"])
def test_golden_novel_2048(lib, merges_path, novel, golden_2048, mode):
    """The reference's committed output for its sample input (348 chunks of 2048 bytes)."""
    gold_ids, gold_off = golden_2048
    t = make_tok(lib, merges_path, 2048)
    m = lib.GTK_MODE_OPT if mode == "opt" else lib.GTK_MODE_BASE
    ids, toff, coff, ms = t.encode(novel, mode=m)
    check_chunks(ids, coff, gold_ids, gold_off, f"golden/{mode}")
    assert toff.tolist() == [0, len(gold_ids)] and ms > 0
    assert t.decode(ids) == novel
    ids2, _, coff2, _ = t.encode(novel, mode=m)           # same handle, second call: identical
    assert np.array_equal(ids, ids2) and np.array_equal(coff, coff2)


@pytest.mark.parametrize("mode", ["opt", "base"])
def test_reference_function_cases(lib, merges_path, ref_cases, mode):
    """Adversarial strings (runs, tiny alphabets, random bytes, UTF-8, empty): one text each."""
    t = make_tok(lib, merges_path, 4096)
    m = lib.GTK_MODE_OPT if mode == "opt" else lib.GTK_MODE_BASE
    blob, case_off = ref_cases["bytes"], ref_cases["case_offsets"]
    ids, toff, coff, _ = t.encode(blob, case_off, mode=m)
    assert np.array_equal(toff, ref_cases["greedy_offsets"]), "per-text offsets"
    assert np.array_equal(ids, ref_cases["greedy_ids"]), first_mismatch(ids, ref_cases["greedy_ids"])
    nonempty = np.flatnonzero(np.diff(case_off) > 0)
    assert len(coff) - 1 == len(nonempty)                 # an empty text owns no chunk


def test_empty_inputs(lib, merges_path):
    t = make_tok(lib, merges_path, 2048)
    ids, toff, coff, ms = t.encode(b"", np.zeros(1, np.int64))
    assert len(ids) == 0 and toff.tolist() == [0] and ms == 0.0
    ids, toff, coff, ms = t.encode(b"", np.zeros(4, np.int64))
    assert len(ids) == 0 and toff.tolist() == [0, 0, 0, 0] and len(coff) == 1
    ids, toff, coff, _ = t.encode_texts([b"", b"a", b"", b" the", b""])
    assert toff.tolist() == [0, 0, 1, 1, 2, 2] and ids[0] == ord("a")


@pytest.mark.parametrize("chunk", [1, 2, 3, 7, 33, 64, 65, 511, 512, 1024, 4095, 4096, 4097, 8192, 32768, 65536])
def test_chunk_sizes_on_novel(lib, merges_path, oracle, novel, chunk):
    t = make_tok(lib, merges_path, chunk)
    data = novel[:40_000] if chunk < 64 else novel[:300_000]
    want, woff = oracle.encode_fixed(data, chunk, mode=MODE_SEGMENTED, threads=NCPU)
    for m in (lib.GTK_MODE_OPT, lib.GTK_MODE_BASE):
        ids, _, coff, _ = t.encode(data, mode=m)
        check_chunks(ids, coff, want, woff, f"chunk {chunk} mode {m}")


def test_config1_correctness_case(lib, merges_path, oracle):
    """1 MiB of seeded text (seed 0), 1024-byte chunks, literal Algorithm 1 on every chunk."""
    data = lib.TextGen(0).text(1 << 20)
    want, woff = oracle.encode_fixed(data, 1024, mode=MODE_GREEDY, threads=NCPU)
    t = make_tok(lib, merges_path, 1024)
    for m in (lib.GTK_MODE_OPT, lib.GTK_MODE_BASE):
        ids, _, coff, _ = t.encode(data, mode=m)
        assert len(coff) - 1 == 1024
        check_chunks(ids, coff, want, woff, f"config1 mode {m}")


def test_config2_full_size(lib, merges_path, oracle):
    """256 MiB (seed 1), 4096-byte chunks: segmented oracle on every chunk, literal oracle on a
    seeded 1 % sample, decode round trip, int64 offsets."""
    n = 256 << 20
    data = lib.TextGen(1).text(n)
    t = make_tok(lib, merges_path, 4096)
    ids, toff, coff, ms = t.encode(data)
    assert len(coff) - 1 == 65536 and coff.dtype == np.int64 and ids.dtype == np.int32
    off = fixed_chunk_offsets(n, 4096)
    want, woff = oracle.encode_chunks(data, off, mode=MODE_SEGMENTED, threads=NCPU)
    check_chunks(ids, coff, want, woff, "config2/all")
    # the literal rule on the seeded 1 % sample (655 chunks; ~40 ms per 4 KiB chunk and core)
    sample = np.sort(np.random.default_rng(1).choice(65536, size=655, replace=False))
    blob = np.concatenate([data[off[c]:off[c + 1]] for c in sample])
    lit, loff = oracle.encode_chunks(blob, np.arange(0, len(blob) + 1, 4096, dtype=np.int64), mode=MODE_GREEDY,
                                     threads=NCPU)
    for k, c in enumerate(sample):
        got, exp = ids[coff[c]:coff[c + 1]], lit[loff[k]:loff[k + 1]]
        assert np.array_equal(got, exp), f"config2 chunk {c}: {first_mismatch(got, exp)}"
    assert t.decode(ids[:coff[256]]) == data[:256 * 4096].tobytes()
    ids_t, _, coff_t, _ = t.encode(data)                # a second run gives the same bits
    assert np.array_equal(ids_t, ids) and np.array_equal(coff_t, coff), "config2: two runs differ"
    lens = np.array([len(oracle.token_bytes(i)) for i in range(oracle.vocab_size)], dtype=np.int64)
    per_chunk = np.add.reduceat(lens[ids], coff[:-1])
    assert np.array_equal(per_chunk, np.diff(off))        # every chunk decodes to exactly its own bytes


def test_config4_long_chunks_unicode_runs(lib, merges_path, oracle):
    """Stress mix (seed 3), 64 MiB in 32 KiB chunks: segmented oracle on all chunks in the fast mode and on
    8 MiB in the one-CTA-per-chunk mode, the literal rule on four chunks (seconds per chunk and core)."""
    n = 64 << 20
    data = lib.TextGen(3).text(n, mix=lib.MIX_STRESS)
    off = fixed_chunk_offsets(n, 32768)
    want, woff = oracle.encode_chunks(data, off, mode=MODE_SEGMENTED, threads=NCPU)
    t = make_tok(lib, merges_path, 32768)
    ids, _, coff, _ = t.encode(data)
    check_chunks(ids, coff, want, woff, "config4/opt")
    ids_b, _, coff_b, _ = t.encode(data[:8 << 20], mode=lib.GTK_MODE_BASE)
    check_chunks(ids_b, coff_b, want[:woff[256]], woff[:257], "config4/base")
    picks = [0, 7, 100, 2047]
    blob = np.concatenate([data[off[c]:off[c + 1]] for c in picks])
    lit, loff = oracle.encode_chunks(blob, np.arange(0, len(blob) + 1, 32768, dtype=np.int64), mode=MODE_GREEDY,
                                     threads=len(picks))
    for k, c in enumerate(picks):
        got, exp = ids[coff[c]:coff[c + 1]], lit[loff[k]:loff[k + 1]]
        assert np.array_equal(got, exp), f"config4 chunk {c} against the literal rule: {first_mismatch(got, exp)}"
    assert t.decode(ids[:coff[8]]) == data[:8 * 32768].tobytes()


def test_config5_lognormal_chunks(lib, merges_path, oracle):
    """Variable-length texts (log-normal, 64 B .. 64 KiB), one chunk each; 512 MiB of the seed-4 text against
    the segmented oracle, a seeded sample of texts against the literal rule."""
    n = 512 << 20
    data = lib.TextGen(4).text(n, mix=lib.MIX_STRESS)
    toff_in = lib.TextGen.lognormal_offsets(4, n)
    want, woff = oracle.encode_chunks(data, toff_in, mode=MODE_SEGMENTED, threads=NCPU)
    t = make_tok(lib, merges_path, 65536)
    ids, toff, coff, _ = t.encode(data, toff_in)
    check_chunks(ids, coff, want, woff, "config5")
    assert np.array_equal(toff, coff)                     # one chunk per text
    lens = np.diff(toff_in)
    rng = np.random.default_rng(4)
    picks = np.sort(np.concatenate([rng.choice(np.flatnonzero(lens <= 4096), 200, replace=False),
                                    rng.choice(np.flatnonzero(lens > 4096), 40, replace=False),
                                    [int(np.argmax(lens)), int(np.argmin(lens))]]))
    blob = np.concatenate([data[toff_in[c]:toff_in[c + 1]] for c in picks])
    boff = np.concatenate([[0], np.cumsum(lens[picks])]).astype(np.int64)
    lit, loff = oracle.encode_chunks(blob, boff, mode=MODE_GREEDY, threads=NCPU)
    for k, c in enumerate(picks):
        got, exp = ids[coff[c]:coff[c + 1]], lit[loff[k]:loff[k + 1]]
        assert np.array_equal(got, exp), f"config5 text {c} ({lens[c]} bytes): {first_mismatch(got, exp)}"


def test_sliced_host_path_boundaries(lib, merges_path, oracle):
    """Host batches of 8 MiB and more are cut into overlapped slices: texts that span slices, empty texts
    at slice edges and a chunk size that divides nothing must give the unsliced result."""
    lens = [30 * (1 << 20) + 11, 0, 5 << 20, 100, 17 * (1 << 20) + 3, 0, 1, 0]
    toff_in = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    data = lib.TextGen(9).text(int(toff_in[-1]), mix=lib.MIX_STRESS)
    t = make_tok(lib, merges_path, 4097)
    ids, toff, coff, ms = t.encode(data, toff_in)
    chunk_off = [0]
    for s, e in zip(toff_in[:-1], toff_in[1:]):
        chunk_off.extend(list(range(int(s) + 4097, int(e), 4097)) + ([int(e)] if e > s else []))
    chunk_off = np.array(chunk_off, np.int64)
    want, woff = oracle.encode_chunks(data, chunk_off, mode=MODE_SEGMENTED, threads=NCPU)
    check_chunks(ids, coff, want, woff, "sliced host path")
    starts = np.searchsorted(chunk_off, toff_in, side="left")
    assert np.array_equal(toff, woff[starts]) and ms > 0
    ids2, toff2, coff2, _ = t.encode(data, toff_in)       # arenas reused: identical on the second call
    assert np.array_equal(ids, ids2) and np.array_equal(coff, coff2) and np.array_equal(toff, toff2)


def test_adversarial_long_segments(lib, merges_path, oracle):
    """Segments far longer than a tile: the whole-CTA path in the HBM workspace."""
    rng = np.random.default_rng(7)
    texts = [b"a" * 65536, b"ab" * 20000, b"e" * 5000 + b" " + b"l" * 9000, ("😀" * 3000).encode(),
             bytes(rng.choice(np.frombuffer(b"ae", np.uint8), size=30000)), b"x" * 4608, b"y" * 4609, b"z" * 4607,
             b"q" * 4096 + b" " + b"w" * 513]
    blob = b"".join(texts)
    toff_in = np.concatenate([[0], np.cumsum([len(x) for x in texts])]).astype(np.int64)
    t = make_tok(lib, merges_path, 65536)
    want, woff = oracle.encode_chunks(blob, toff_in, mode=MODE_SEGMENTED, threads=NCPU)
    for m in (lib.GTK_MODE_OPT, lib.GTK_MODE_BASE):
        ids, toff, coff, _ = t.encode(blob, toff_in, mode=m)
        check_chunks(ids, coff, want, woff, f"long segments mode {m}")
    lit, _ = oracle.encode_chunks(blob, toff_in[:2], mode=MODE_GREEDY)
    assert np.array_equal(want[:woff[1]], lit)            # 64 Ki of 'a': the literal rule agrees


def test_long_and_huge_segments_in_a_large_batch(lib, merges_path, oracle):
    """Segments of every class -- one thread's, a warp's, and ones far longer than a tile that the whole CTA
    finishes in the workspace -- inside a 12 MiB host batch (which the host path cuts into slices)."""
    rng = np.random.default_rng(3)
    filler = lib.TextGen(8).text(12 << 20, mix=lib.MIX_STRESS).copy()
    inserts = [b"a" * 65536, b"ab" * 1500, ("\u65e5" * 900).encode(), b"e" * 2048, b"e" * 2049, b"l" * 33, b"s" * 32,
               b"x" * 5000 + b" " + b"y" * 4608, bytes(rng.choice(np.frombuffer(b"ae", np.uint8), size=20000))]
    pos = 1 << 20
    for blob in inserts:
        filler[pos:pos + len(blob)] = np.frombuffer(blob, np.uint8)
        pos += len(blob) + (1 << 20) + 12345
    lens = [3 << 20, 65536, 0, (5 << 20) + 17, len(filler) - (3 << 20) - 65536 - (5 << 20) - 17]
    toff_in = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    t = make_tok(lib, merges_path, 65536)
    chunk_off = [0]
    for s, e in zip(toff_in[:-1], toff_in[1:]):
        chunk_off.extend(list(range(int(s) + 65536, int(e), 65536)) + ([int(e)] if e > s else []))
    want, woff = oracle.encode_chunks(filler, np.array(chunk_off, np.int64), mode=MODE_SEGMENTED, threads=NCPU)
    ids, toff, coff, _ = t.encode(filler, toff_in)
    check_chunks(ids, coff, want, woff, "all segment classes")
    assert t.decode(ids[:coff[20]]) == filler[:chunk_off[20]].tobytes()


def test_crowded_pair_bucket(lib, merges_path, tmp_path):
    """More than four pairs in one bucket of the device pair table: the fifth and later ones are found in
    the side table (second load), in every kernel that probes."""
    from conftest import crowded_bucket_merges
    from oracle.loader import Oracle

    path = str(tmp_path / "crowded_merges.txt")
    text, n_second = crowded_bucket_merges(merges_path, path)
    data = np.frombuffer(text, np.uint8)
    want, woff = Oracle(path).encode_fixed(data, 512)
    assert (want >= 1280).sum() > 100
    t = lib.Tokenizer(path, 512, 50, device=0)
    assert t.table_info()["hash_overflow_entries"] >= 2
    for mode in (lib.GTK_MODE_OPT, lib.GTK_MODE_BASE):
        ids, _, coff, _ = t.encode(data, mode=mode)
        check_chunks(ids, coff, want, woff, f"crowded bucket, mode {mode}")
    big = np.tile(data, 40)  # a batch large enough for the multi-CTA tile kernel (not the single-CTA path)
    want, woff = Oracle(path).encode_fixed(big, 512, threads=NCPU)
    ids, _, coff, _ = t.encode(big)
    check_chunks(ids, coff, want, woff, "crowded bucket, tiled")


def test_irregular_table(lib, merges_path, novel, tmp_path):
    """A table that is not monotone and whose merged ids are not 256 + rank: the pass kernels merge one
    occurrence per pass, merged ids come from the per-rank array, every mode and every batch path."""
    from conftest import irregular_merges
    from oracle.loader import MODE_LOCALMIN, Oracle

    path = str(tmp_path / "irregular_merges.txt")
    irregular_merges(merges_path, path)
    orc = Oracle(path)
    t = lib.Tokenizer(path, 1000, 50, device=0)
    ti = t.table_info()
    assert ti["monotone"] == 0 and ti["merged_is_256_plus_rank"] == 0
    stress = lib.TextGen(7).text(1 << 20, mix=lib.MIX_STRESS)
    for name, data in (("novel", np.frombuffer(novel[:300_000], np.uint8)), ("stress", stress)):
        want, woff = orc.encode_fixed(data, 1000, threads=NCPU)
        for mode in (lib.GTK_MODE_OPT, lib.GTK_MODE_BASE):
            ids, _, coff, _ = t.encode(data, mode=mode)
            check_chunks(ids, coff, want, woff, f"irregular table, {name}, mode {mode}")
    small = np.frombuffer(novel[5000:9000], np.uint8)  # single-CTA path
    want, woff = orc.encode_fixed(small, 1000)
    ids, _, coff, _ = t.encode(small)
    check_chunks(ids, coff, want, woff, "irregular table, small batch")
    want, woff = orc.encode_fixed(small, 1000, mode=MODE_LOCALMIN)
    ids, _, coff, _ = t.encode(small, mode=lib.GTK_MODE_LOCALMIN)
    check_chunks(ids, coff, want, woff, "irregular table, local-minimum rule")


def test_random_small_batches(lib, merges_path, oracle):
    """Many short texts of assorted lengths in one batch (latency-mode strings, ragged)."""
    rng = np.random.default_rng(11)
    src = lib.TextGen(2).text(4 << 20, mix=lib.MIX_STRESS)
    lens = rng.integers(0, 1500, size=3000)
    lens[::97] = 0
    toff_in = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    data = src[:toff_in[-1]]
    t = make_tok(lib, merges_path, 512)
    ids, toff, coff, _ = t.encode(data, toff_in)
    chunk_off = [0]
    for s, e in zip(toff_in[:-1], toff_in[1:]):
        chunk_off.extend(list(range(int(s) + 512, int(e), 512)) + ([int(e)] if e > s else []))
    want, woff = oracle.encode_chunks(data, np.array(chunk_off, np.int64), mode=MODE_SEGMENTED, threads=NCPU)
    check_chunks(ids, coff, want, woff, "ragged batch")
    starts = np.searchsorted(np.array(chunk_off), toff_in, side="left")
    assert np.array_equal(toff, woff[starts])


def test_medium_batches_of_many_short_texts(lib, merges_path, oracle):
    """Batches of thousands of short texts, which the single-CTA chunker lays out per text: only one-chunk and
    empty texts; a few texts of more than 32 chunks among them (one warp each, from the list in shared
    memory); more such texts than that list holds (the scan over all texts).  Host and device-resident entry."""
    import torch

    rng = np.random.default_rng(31)
    src = lib.TextGen(6).text(2 << 20, mix=lib.MIX_STRESS)
    cases = []
    lens = rng.integers(0, 100, size=9000)
    lens[::53] = 0
    cases.append(("short only", 2048, lens))
    lens = rng.integers(0, 60, size=5000)
    lens[[7, 2500, 4999]] = [64 * 40 + 3, 64 * 33, 64 * 200 + 1]
    cases.append(("a few long texts", 64, lens))
    lens = np.full(7000, 4)
    lens[rng.choice(7000, size=140, replace=False)] = 16 * 34 - 5
    cases.append(("more long texts than the list holds", 16, lens))
    for what, chunk, lens in cases:
        toff_in = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        n = int(toff_in[-1])
        assert n // chunk <= len(lens) and n > 32768           # the shape the per-text layout is chosen for
        data = src[:n]
        chunk_off = [0]
        for s, e in zip(toff_in[:-1], toff_in[1:]):
            chunk_off.extend(list(range(int(s) + chunk, int(e), chunk)) + ([int(e)] if e > s else []))
        chunk_off = np.array(chunk_off, np.int64)
        want, woff = oracle.encode_chunks(data, chunk_off, mode=MODE_SEGMENTED, threads=NCPU)
        starts = np.searchsorted(chunk_off, toff_in, side="left")
        t = make_tok(lib, merges_path, chunk)
        ids, toff, coff, _ = t.encode(data, toff_in)
        check_chunks(ids, coff, want, woff, what)
        assert np.array_equal(toff, woff[starts]), what
        d_bytes, d_toff = torch.from_numpy(data.copy()).cuda(), torch.from_numpy(toff_in).cuda()
        d_ids = torch.empty(n, dtype=torch.int32, device="cuda")
        d_coff = torch.empty(len(chunk_off) + 8, dtype=torch.int64, device="cuda")
        n_ids, n_chunks, _ = t.encode_device(d_bytes.data_ptr(), n, d_toff.data_ptr(), len(lens), d_ids.data_ptr(), n,
                                             d_coff.data_ptr(), d_coff.numel())
        assert n_chunks == len(woff) - 1 and n_ids == len(want), what
        assert np.array_equal(d_ids[:n_ids].cpu().numpy(), want), what
        assert np.array_equal(d_coff[:n_chunks + 1].cpu().numpy(), woff), what
        assert t.stage_ms()["kernel_launches"] == 4, what        # chunker, merge, scans, pack: one launch each


def test_path_selector_boundaries(lib, merges_path, oracle):
    """Batches on both sides of every size limit that picks a code path: the single-CTA chunker by search (256
    texts, 2048 chunks, 1024 tiles) and per text (16 384 items, 2048 tiles), the single-CTA scans (16 384 items), the
    small-batch kernel (8 KiB, 1024 texts), the two-launch path (64 KiB, 1024 texts, 4096 chunks) and the sliced
    host path (8 MiB).  Host and device-resident entry."""
    import torch

    src = lib.TextGen(8).text(9 << 20, mix=lib.MIX_STRESS)

    def check(what, chunk, lens, host=True):
        lens = np.asarray(lens, dtype=np.int64)
        toff_in = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        n = int(toff_in[-1])
        data = src[:n]
        ends = toff_in[1:]
        inner = [np.arange(s + chunk, e, chunk) for s, e in zip(toff_in[:-1], ends) if e - s > chunk]
        chunk_off = np.unique(np.concatenate([[0], ends[lens > 0]] + inner)).astype(np.int64)
        want, woff = oracle.encode_chunks(data, chunk_off, mode=MODE_SEGMENTED, threads=NCPU)
        starts = np.searchsorted(chunk_off, toff_in, side="left")
        t = make_tok(lib, merges_path, chunk)
        if host:
            ids, toff, coff, _ = t.encode(data, toff_in)
            check_chunks(ids, coff, want, woff, what + " (host)")
            assert np.array_equal(toff, woff[starts]), what
        d_bytes, d_toff = torch.from_numpy(data.copy()).cuda(), torch.from_numpy(toff_in).cuda()
        d_ids = torch.empty(n, dtype=torch.int32, device="cuda")
        d_coff = torch.empty(len(chunk_off) + 8, dtype=torch.int64, device="cuda")
        n_ids, n_chunks, _ = t.encode_device(d_bytes.data_ptr(), n, d_toff.data_ptr(), len(lens), d_ids.data_ptr(), n,
                                             d_coff.data_ptr(), d_coff.numel())
        assert n_chunks == len(woff) - 1 and n_ids == len(want), what
        assert np.array_equal(d_ids[:n_ids].cpu().numpy(), want), what
        assert np.array_equal(d_coff[:n_chunks + 1].cpu().numpy(), woff), what
        return t.stage_ms()["kernel_launches"]

    # chunker by search: 256 / 257 texts of ~3 chunks; 2048 / 2049 as the bound on chunks; 1024 / 1025 tiles
    assert check("256 texts", 512, [1300] * 256) == 4
    assert check("257 texts", 512, [1300] * 257) > 4
    assert check("chunk bound 2048", 512, [2046 * 512]) == 4
    assert check("chunk bound 2049", 512, [2047 * 512]) > 4
    assert check("1024 tiles", 4096, [1024 * 4096]) == 4
    assert check("1025 tiles", 4096, [1024 * 4096 + 1]) >= 4
    # chunker per text and the scans: the bound on chunks (bytes / chunk + texts + 1) at 16 384 / 16 386
    assert check("16 376 as the chunk bound", 128, [3] * 16000) == 4
    assert check("16 386 as the chunk bound", 128, [3] * 16010) > 4
    # per text: 2048 / 2049 tiles (8 MiB: device-resident entry only, the host entry slices such a batch)
    assert check("2048 tiles, many texts", 4096, [1024] * 8192, host=False) == 4
    assert check("2049 tiles, many texts", 4096, [1024] * 8192 + [1], host=False) > 4
    # small-batch kernel: 8 KiB / one byte more; 1024 / 1025 texts
    check("8 KiB", 2048, [8192])
    check("8 KiB + 1", 2048, [8193])
    check("16 KiB", 2048, [16384])
    check("32 KiB", 2048, [32768])
    check("1024 texts", 2048, [20] * 1024)
    check("1025 texts", 2048, [20] * 1025)
    # several texts in two launches (host entry): up to 64 KiB, 1024 texts and 4096 chunks
    check("50 texts of 1000 bytes", 300, [1000] * 50)
    check("1024 short texts, some empty", 64, [60, 0, 61, 59] * 256)
    check("1025 short texts", 64, [60] * 1025)
    check("ragged texts across tiles", 4096, [5000, 1, 0, 4095, 4097, 8192, 12000, 3])
    # one text in two launches (host entry): up to 64 KiB and 4096 chunks
    check("64 KiB", 2048, [65536])
    check("64 KiB + 1", 2048, [65537])
    check("64 KiB in 4096 chunks", 16, [65536])
    check("40 000 bytes in 5715 chunks", 7, [40000])
    check("one text of 50 000 bytes, chunk longer than the text", 65536, [50000])
    t = make_tok(lib, merges_path, 1000)                      # ... and in GPT-2's id space
    ref, _, _, _ = t.encode(src[:60000])
    t.set_id_space(True)
    ids, _, _, _ = t.encode(src[:60000])
    gpt2_of_byte = {b: i for i, b in enumerate(list(range(33, 127)) + list(range(161, 173)) + list(range(174, 256)))}
    nxt = 188
    for b in range(256):
        if b not in gpt2_of_byte:
            gpt2_of_byte[b] = nxt
            nxt += 1
    lut = np.arange(65536, dtype=np.int32)
    lut[:256] = [gpt2_of_byte[b] for b in range(256)]
    assert np.array_equal(ids, lut[ref])
    # sliced host path: one byte below and at 8 MiB
    check("8 MiB - 1", 4096, [(8 << 20) - 1])
    check("8 MiB", 4096, [8 << 20])


def test_interleaved_paths_on_one_handle(lib, merges_path, oracle):
    """One handle, calls of every kind in turn -- single-kernel, single-piece, sliced, device-resident, host reference,
    empty -- twice over: each result must be that call's own (the result views, arenas and flags of one path must
    not leak into the next)."""
    import torch

    src = lib.TextGen(12).text(10 << 20, mix=lib.MIX_STRESS)
    rng = np.random.default_rng(5)
    t = make_tok(lib, merges_path, 1024)

    def offsets(lens):
        return np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)

    def expected(data, toff_in):
        ends = toff_in[1:]
        lens = np.diff(toff_in)
        inner = [np.arange(s + 1024, e, 1024) for s, e in zip(toff_in[:-1], ends) if e - s > 1024]
        chunk_off = np.unique(np.concatenate([[0], ends[lens > 0]] + inner)).astype(np.int64)
        want, woff = oracle.encode_chunks(data, chunk_off, mode=MODE_SEGMENTED, threads=NCPU)
        return want, woff, woff[np.searchsorted(chunk_off, toff_in, side="left")]

    batches = {
        "single kernel": offsets([300, 0, 212]),
        "single piece, one text": offsets([200_000]),
        "one text in two launches": offsets([40_000]),
        "single piece, many texts": offsets(rng.integers(0, 90, size=6000)),
        "sliced": offsets([5 << 20, 0, (4 << 20) + 77]),
    }
    want = {k: expected(src[:v[-1]], v) for k, v in batches.items()}
    order = ["sliced", "one text in two launches", "single kernel", "single piece, many texts", "single piece, one text",
             "one text in two launches", "single kernel"]
    for rnd in range(2):
        for k in order:
            toff_in = batches[k]
            data = src[:toff_in[-1]]
            ids, toff, coff, _ = t.encode(data, toff_in)
            w, woff, wtext = want[k]
            check_chunks(ids, coff, w, woff, f"{k}, round {rnd}")
            assert np.array_equal(toff, wtext), k
            if k == "single piece, one text":               # the device-resident entry and the host reference in between
                d_bytes, d_toff = torch.from_numpy(data.copy()).cuda(), torch.from_numpy(toff_in).cuda()
                d_ids = torch.empty(len(data), dtype=torch.int32, device="cuda")
                n_ids, n_chunks, _ = t.encode_device(d_bytes.data_ptr(), len(data), d_toff.data_ptr(), 1,
                                                     d_ids.data_ptr(), len(data))
                assert n_ids == len(w) and np.array_equal(d_ids[:n_ids].cpu().numpy(), w)
                cids, _, ccoff = t.encode_cpu(data[:5000], None)[:3]         # its first four chunks are the batch's
                assert np.array_equal(cids[:ccoff[4]], w[:woff[4]]) and len(ccoff) == 6
                eids, etoff, ecoff, _ = t.encode(np.zeros(0, np.uint8), np.array([0, 0, 0], dtype=np.int64))
                assert len(eids) == 0 and np.array_equal(etoff, [0, 0, 0])


def test_generated_adversarial_strings(lib, merges_path, oracle):
    """Seeded adversarial strings (runs, tiny alphabets, arbitrary bytes, multi-byte characters, empty) in
    batches that take the single-kernel small path and the multi-kernel path, at several chunk sizes."""
    rng = np.random.default_rng(21)
    alphabets = [b"a", b"ab", b"ae l", b"\n", bytes(range(256)), "\u00e9\u65e5\U0001F600 x".encode(), b"the and ing tion ", b" \t.,"]
    texts = []
    for i in range(600):
        alpha = np.frombuffer(alphabets[i % len(alphabets)], dtype=np.uint8)
        texts.append(bytes(rng.choice(alpha, size=int(rng.integers(0, 200)))))
    for chunk in (5, 64, 2048):
        t = make_tok(lib, merges_path, chunk)
        for batch in (texts[:40], texts):                                  # small path, general path
            ids, toff, coff, _ = t.encode_texts(batch)
            blob = b"".join(batch)
            chunk_off = [0]
            pos = 0
            for x in batch:
                chunk_off.extend(list(range(pos + chunk, pos + len(x), chunk)) + ([pos + len(x)] if x else []))
                pos += len(x)
            want, woff = oracle.encode_chunks(blob, np.array(chunk_off, np.int64), mode=MODE_GREEDY)
            check_chunks(ids, coff, want, woff, f"generated strings, chunk {chunk}, {len(batch)} texts")


def test_latency_strings_one_call_each(lib, merges_path, oracle):
    """Config 3: 10 000 independent 512-byte strings (seed 2), one call each with batch size 1, every string
    checked against the literal rule."""
    count = 10000
    data = lib.TextGen(2).blocks(count, 512)
    off = np.arange(0, count * 512 + 1, 512, dtype=np.int64)
    want, woff = oracle.encode_chunks(data, off, mode=MODE_GREEDY, threads=NCPU)
    t = make_tok(lib, merges_path, 2048)
    for i in range(count):
        ids, _, coff, _ = t.encode(data[off[i]:off[i + 1]])
        exp = want[woff[i]:woff[i + 1]]
        assert len(coff) == 2 and np.array_equal(ids, exp), f"string {i}: {first_mismatch(ids, exp)}"


def test_device_resident_entry_point(lib, merges_path, oracle):
    import torch

    data = lib.TextGen(1).text(8 << 20)
    n = len(data)
    d_bytes = torch.from_numpy(data.copy()).cuda()
    d_toff = torch.tensor([0, n], dtype=torch.int64, device="cuda")
    d_ids = torch.empty(n, dtype=torch.int32, device="cuda")
    d_coff = torch.empty(n // 4096 + 8, dtype=torch.int64, device="cuda")
    t = make_tok(lib, merges_path, 4096)
    n_ids, n_chunks, ms = t.encode_device(d_bytes.data_ptr(), n, d_toff.data_ptr(), 1, d_ids.data_ptr(), n,
                                          d_coff.data_ptr(), d_coff.numel())
    want, woff = oracle.encode_fixed(data, 4096, mode=MODE_SEGMENTED, threads=NCPU)
    assert n_chunks == 2048 and n_ids == len(want) and ms > 0
    assert np.array_equal(d_ids[:n_ids].cpu().numpy(), want)
    assert np.array_equal(d_coff[:n_chunks + 1].cpu().numpy(), woff)
    st = t.stage_ms()                                     # by default only the pipeline as a whole is timed
    assert st["kernel_launches"] >= 4 and st["merge"] == 0 and st["pipeline"] == pytest.approx(ms)
    t.set_stage_timing(True)
    _, _, ms2 = t.encode_device(d_bytes.data_ptr(), n, d_toff.data_ptr(), 1, d_ids.data_ptr(), n,
                                d_coff.data_ptr(), d_coff.numel())
    st = t.stage_ms()
    assert 0 < st["merge"] < st["pipeline"] == pytest.approx(ms2) and st["pack"] > 0 and st["chunker"] > 0
    assert np.array_equal(d_ids[:n_ids].cpu().numpy(), want)
    with pytest.raises(lib.GtkError) as e:                # too small an id buffer is reported, not overrun
        t.encode_device(d_bytes.data_ptr(), n, d_toff.data_ptr(), 1, d_ids.data_ptr(), 1000)
    assert e.value.code == 4


def test_batch_beyond_2_gib_uses_64_bit_offsets(lib, merges_path, oracle):
    """2.25 GiB in one call (byte positions and id offsets beyond 2^31): every chunk must decode to exactly its own
    bytes (token byte lengths summed per chunk), a seeded sample of chunks must equal the oracle, and the
    device-resident entry point must agree with the host path."""
    import torch

    n = (9 << 28) + 4096 * 3 + 17
    data = lib.TextGen(11).text(n)
    t = make_tok(lib, merges_path, 4096)
    ids, toff, coff, _ = t.encode(data)
    n_chunks = (n + 4095) // 4096
    assert len(coff) - 1 == n_chunks and toff.tolist() == [0, len(ids)] and coff[-1] == len(ids)
    lens = np.array([len(oracle.token_bytes(i)) for i in range(oracle.vocab_size)], dtype=np.int64)
    per_chunk = np.add.reduceat(lens[ids], coff[:-1])
    want_len = np.full(n_chunks, 4096, dtype=np.int64)
    want_len[-1] = n - 4096 * (n_chunks - 1)
    assert np.array_equal(per_chunk, want_len)
    rng = np.random.default_rng(2)
    sample = np.unique(np.concatenate([rng.integers(0, n_chunks, size=400), [0, n_chunks - 1, (1 << 31) // 4096,
                                                                            (1 << 31) // 4096 - 1]]))
    for c in sample:
        lo, hi = int(c) * 4096, min(int(c) * 4096 + 4096, n)
        want, _ = oracle.encode_chunks(data[lo:hi], np.array([0, hi - lo]), mode=MODE_SEGMENTED)
        assert np.array_equal(ids[coff[c]:coff[c + 1]], want), f"chunk {c}"
    d_bytes = torch.from_numpy(data).cuda()
    d_toff = torch.tensor([0, n], dtype=torch.int64, device="cuda")
    d_ids = torch.empty(len(ids) + 16, dtype=torch.int32, device="cuda")
    d_coff = torch.empty(n_chunks + 8, dtype=torch.int64, device="cuda")
    n_ids, n_c, _ = t.encode_device(d_bytes.data_ptr(), n, d_toff.data_ptr(), 1, d_ids.data_ptr(), d_ids.numel(),
                                    d_coff.data_ptr(), d_coff.numel())
    assert n_ids == len(ids) and n_c == n_chunks
    assert torch.equal(d_ids[:n_ids].cpu(), torch.from_numpy(ids))
    assert torch.equal(d_coff[:n_c + 1].cpu(), torch.from_numpy(coff))


def test_invalid_arguments_are_reported(lib, merges_path):
    t = make_tok(lib, merges_path, 2048)
    with pytest.raises(lib.GtkError) as e:
        t.encode(b"abcdef", np.array([0, 4, 2, 6], dtype=np.int64))      # offsets must not decrease
    assert e.value.code == 1
    with pytest.raises(lib.GtkError) as e:
        t.encode(b"abcdef", np.array([1, 6], dtype=np.int64))            # first offset must be 0
    assert e.value.code == 1
    with pytest.raises(lib.GtkError) as e:
        t.encode(b"abc", mode=7)
    assert e.value.code == 1
    ids, _, _, _ = t.encode(b"abc")                                       # the handle stays usable
    assert len(ids) >= 1


def test_localmin_rule_on_gpu(lib, merges_path, oracle, novel, ref_cases):
    """GTK_MODE_LOCALMIN: the reference's other merge rule (bpe_merge_kernel_optimized), per chunk, capped at
    max_iters passes -- against the oracle's restatement of bpe_merge_cpu (pinned by the reference's
    gpu_tokens_optimized.txt) and the outputs recorded from the reference's compiled function."""
    from oracle.loader import MODE_LOCALMIN

    t = make_tok(lib, merges_path, 4096)
    blob, case_off = ref_cases["bytes"], ref_cases["case_offsets"]
    ids, toff, _, _ = t.encode(blob, case_off, mode=lib.GTK_MODE_LOCALMIN)
    assert np.array_equal(toff, ref_cases["localmin_offsets"])
    assert np.array_equal(ids, ref_cases["localmin_ids"]), first_mismatch(ids, ref_cases["localmin_ids"])
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_localmin_512.npz"))
    ids, _, _, _ = t.encode(z["text"], mode=lib.GTK_MODE_LOCALMIN)
    assert np.array_equal(ids, z["ids"])
    for data, chunk in ((novel[:400_000], 2048), (lib.TextGen(3).text(3 << 20, mix=lib.MIX_STRESS), 32768),
                        (b"a" * 70000 + b" " + b"ab" * 5000, 65536)):
        t = make_tok(lib, merges_path, chunk)
        off = fixed_chunk_offsets(len(data), chunk)
        want, woff = oracle.encode_chunks(data, off, mode=MODE_LOCALMIN, max_iters=50, threads=NCPU)
        ids, _, coff, ms = t.encode(data, mode=lib.GTK_MODE_LOCALMIN)
        check_chunks(ids, coff, want, woff, f"localmin chunk {chunk}")
        greedy, _, _, _ = t.encode(data)
        assert len(greedy) <= len(ids)                    # the capped local-minimum rule never merges more


def test_gpt2_id_space(lib, merges_path, oracle):
    """Optional output in GPT-2's own id space: ids < 256 move to their position in GPT-2's byte-symbol order,
    ids >= 256 are unchanged."""
    t = make_tok(lib, merges_path, 2048)
    ref_ids, _, _, _ = t.encode(b"Hello world")
    t.set_id_space(True)
    ids, _, _, _ = t.encode(b"Hello world")
    assert ids.tolist() == [15496, 995] == ref_ids.tolist()          # whole-word tokens: same in both spaces
    raw = bytes(range(256)) + b" \n!~"
    ids, _, _, _ = t.encode(raw)
    t.set_id_space(False)
    ref, _, _, _ = t.encode(raw)
    order = [b for b in range(256) if 33 <= b <= 126 or 161 <= b <= 172 or 174 <= b <= 255]
    order += [b for b in range(256) if b not in order]                # GPT-2 bytes_to_unicode order
    gpt2_of_byte = {b: i for i, b in enumerate(order)}
    want = [gpt2_of_byte[x] if x < 256 else x for x in ref.tolist()]
    assert ids.tolist() == want
    assert gpt2_of_byte[0x20] == 220 and gpt2_of_byte[ord("!")] == 0 and gpt2_of_byte[0] == 188
    big = lib.TextGen(5).text(6 << 20, mix=lib.MIX_STRESS)            # multi-kernel path as well
    ref, _, _, _ = t.encode(big)
    t.set_id_space(True)
    ids, _, _, _ = t.encode(big)
    lut = np.arange(65536, dtype=np.int32)
    lut[:256] = [gpt2_of_byte[b] for b in range(256)]
    assert np.array_equal(ids, lut[ref])


def test_standalone_cli_reproduces_reference_run(native_built, merges_path, novel, tmp_path):
    """The command-line front end: reference argv, reference stdout lines (the regex of
    benchmark_tokenizer_scaling.py:155-157 must match), exit code 0 on CPU == GPU, and an output file
    with the sha256 of the reference's committed data/output/gpu_tokens_blockbpe.txt."""
    import hashlib
    import json
    import re
    import subprocess

    from conftest import GOLDEN

    text = tmp_path / "novel.txt"
    text.write_bytes(novel)
    out = tmp_path / "tokens.txt"
    env = dict(os.environ, GTK_MERGES=merges_path, GTK_OUTPUT=str(out))
    want = json.load(open(os.path.join(GOLDEN, "MANIFEST.json")))["sources"]["data/output/gpu_tokens_blockbpe.txt"]
    for extra in ([], ["opt"]):
        r = subprocess.run([native_built.CLI, "2048", str(text)] + extra, env=env, capture_output=True, text=True,
                           timeout=300)
        assert r.returncode == 0, r.stderr
        m = re.search(r"GPU BlockBPE-style greedy kernel time.*:\s*([0-9.]+)\s*ms", r.stdout)
        assert m and float(m.group(1)) > 0
        assert "CPU vs GPU token match (greedy Algorithm 1): OK" in r.stdout
        assert "Loaded BPE merges: 50000, vocab size: 50256" in r.stderr
        assert "Tokenized full text into 348 chunk(s), max tokens per chunk: 2048" in r.stderr
        assert hashlib.sha256(out.read_bytes()).hexdigest() == want


def test_base_kernel_block_sizes(lib, native_built, merges_path, novel, oracle, tmp_path):
    """The reference's BLOCK_SIZE sweep (profile_blockbpe_block_sizes.sh:9-10,22-25) as a run-time setting: every
    block size gives the ids of the literal rule at every chunk length, other sizes are refused, and the sweep
    script prints the reference's CSV columns."""
    import subprocess

    text = np.frombuffer(novel[:200_000], dtype=np.uint8)
    for chunk in (128, 1024, 4096):
        want, woff = oracle.encode_fixed(novel[:200_000], chunk, mode=MODE_GREEDY, threads=os.cpu_count() or 1)
        t = make_tok(lib, merges_path, chunk)
        for threads in (0, 64, 128, 256, 512, 1024):
            t.set_base_block_size(threads)
            ids, _, coff, ms = t.encode(text, mode=lib.GTK_MODE_BASE)
            assert np.array_equal(ids, want) and np.array_equal(coff, woff), (chunk, threads)
            assert ms > 0
        with pytest.raises(lib.GtkError):
            t.set_base_block_size(96)
    big = make_tok(lib, merges_path, 32768)                      # a small CTA on a chunk far beyond its warp count
    stress = lib.TextGen(3).text(1 << 20, mix=lib.MIX_STRESS)
    ref, _, roff, _ = big.encode(stress, mode=lib.GTK_MODE_OPT)
    big.set_base_block_size(128)
    ids, _, coff, _ = big.encode(stress, mode=lib.GTK_MODE_BASE)
    assert np.array_equal(ids, ref) and np.array_equal(coff, roff)

    src = tmp_path / "novel.txt"
    src.write_bytes(novel[:100_000])
    env = dict(os.environ, GTK_MERGES=merges_path, GTK_OUTPUT=str(tmp_path / "tokens.txt"))
    script = os.path.join(os.path.dirname(native_built.CLI), "profile_blockbpe_block_sizes.sh")
    r = subprocess.run(["bash", script, str(src)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    rows = [ln.split(",") for ln in r.stdout.splitlines() if ln[:1].isdigit()]
    assert "block_size,seq_len,cpu_ms,gpu_ms,gpu_tokens_per_s" in r.stdout
    assert len(rows) == 24 and {row[0] for row in rows} == {"128", "256", "512", "1024"}
    assert all(len(row) == 5 and float(row[3]) > 0 and float(row[4]) > 0 for row in rows)


def test_pybind_methods_on_gpu(lib, merges_path, oracle):
    import gputok_gpu

    tok = gputok_gpu.GpuTokenizer(merges_path, 2048, 50)
    texts = ["Hello world!", "", "The weather today is", "naïve café 日本 " * 300]
    for method in (tok.tokenize_batch, tok.tokenize_batch_blockbpe_base):
        batch, ms = method(texts)
        assert len(batch) == 4 and batch[1] == [] and ms > 0
        for text, ids in zip(texts, batch):
            want, _ = oracle.encode_fixed(text.encode(), 2048, mode=MODE_GREEDY)
            assert ids == want.tolist()
    assert tok.tokenize_batch([]) == ([], 0.0)
    assert tok.tokenize_batch(["", ""]) == ([], 0.0)     # all-empty batch, as the reference
    assert tok.tokenize_batch_cpu(texts) == tok.tokenize_batch(texts)[0]
    lm_gpu, _ = tok.tokenize_batch(texts[:3], merge_rule="localmin")      # texts shorter than a chunk
    assert lm_gpu == tok.tokenize_batch_cpu(texts[:3], merge_rule="localmin")
    ids, toff, coff, ms = tok.encode_packed(texts)
    assert ids.dtype == np.int32 and toff.dtype == np.int64 and toff[-1] == len(ids)


def test_stage_times_of_a_sliced_batch(lib, merges_path):
    """A host batch large enough to be cut into slices reports the stage times of all its slices: the merge
    time must be close to the device-resident figure for the same bytes, not that of one slice."""
    import torch

    n = 96 << 20
    data = lib.TextGen(1).text(n)
    t = make_tok(lib, merges_path, 4096)
    t.encode(data)
    t.encode(data)
    sliced = t.stage_ms()
    d_bytes = torch.from_numpy(data).cuda()
    d_toff = torch.tensor([0, n], dtype=torch.int64, device="cuda")
    d_ids = torch.empty(n, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    t.set_stage_timing(True)
    for _ in range(2):
        t.encode_device(d_bytes.data_ptr(), n, d_toff.data_ptr(), 1, d_ids.data_ptr(), n)
    whole = t.stage_ms()
    assert whole["merge"] > 0
    assert 0.7 * whole["merge"] < sliced["merge"] < 2.5 * whole["merge"], (sliced, whole)
    assert sliced["pipeline"] >= sliced["merge"] and sliced["pack"] > 0


def test_two_devices_two_threads_one_process(lib, merges_path, oracle):
    """One handle per GPU, driven from two threads of one process: a 64 MiB batch of log-normal texts is cut
    into two byte ranges, each range is tokenised on its own device, the offsets are stitched on the host and
    the whole equals the oracle on the unsplit batch."""
    import threading

    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    n = 64 << 20
    data = lib.TextGen(4).text(n, mix=lib.MIX_STRESS)
    toff_in = lib.TextGen.lognormal_offsets(4, n)
    bounds = lib.partition_by_bytes(toff_in, 2)
    results, errors = [None, None], []

    def work(dev):
        try:
            lo, hi = int(bounds[dev]), int(bounds[dev + 1])
            tok = lib.Tokenizer(merges_path, 65536, 50, device=dev)
            part = data[toff_in[lo]:toff_in[hi]]
            for _ in range(3):                              # repeated calls while the other thread runs too
                ids, toff, coff, _ = tok.encode(part, toff_in[lo:hi + 1] - toff_in[lo])
            results[dev] = (ids, coff)
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(d,)) for d in (0, 1)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    ids = np.concatenate([results[0][0], results[1][0]])
    coff = lib.stitch_offsets([results[0][1], results[1][1]])
    want, woff = oracle.encode_chunks(data, toff_in, mode=MODE_SEGMENTED, threads=NCPU)
    check_chunks(ids, coff, want, woff, "two devices")


def test_checked_build_runs_clean(native_built):
    """The library built with -DGTK_CHECKED (every data-dependent index into shared memory, the lane scratch,
    the staging buffer and the count arrays is compared with its limit; a violation is recorded and the
    access skipped) runs the golden, config-1, adversarial-segment and irregular-table tests in a process of
    its own and must end with an empty record.  The mechanism itself is exercised first: a check that is
    made to fail is reported with its id, value and limit, and nothing faults."""
    import ctypes
    import subprocess
    import sys

    from gputok_b200.capi import checked_library_path

    path = checked_library_path()
    assert os.path.exists(path), "the checked build is part of build_all()"
    probe = ("import ctypes,sys; lib=ctypes.CDLL(sys.argv[1]); w=(ctypes.c_int*4)(); "
             "rc=lib.gtk_debug_check_words(w,1,1); print('SELFTEST',rc,w[0],w[1],w[2],w[3]); "
             "rc=lib.gtk_debug_check_words(w,0,0); print('AFTER_RESET',rc,w[3])")
    out = subprocess.run([sys.executable, "-c", probe, path], capture_output=True, text=True, timeout=300)
    assert "SELFTEST 0 99 5 4 1" in out.stdout and "AFTER_RESET 0 0" in out.stdout, out.stdout + out.stderr
    env = dict(os.environ, GPUTOK_B200_LIBRARY=path)
    here = os.path.dirname(os.path.abspath(__file__))
    sel = ("golden_novel or reference_function_cases or config1 or adversarial_long_segments or "
           "long_and_huge_segments or irregular_table or crowded_pair_bucket or random_small_batches or chunk_sizes")
    run = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_gpu_parity.py"), "-m", "gpu", "-x",
                          "-q", "-s", "-k", sel], capture_output=True, text=True, timeout=1500, env=env)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-2000:]
    assert "CHECKED_BUILD rc=0 failures=0" in run.stdout, run.stdout[-2000:]


def test_merge_table_beyond_16_bits(lib, merges_path, oracle, novel, tmp_path):
    """A merges file with 66 000 merges (ids and ranks beyond 16 bits): the reference accepts any file, and so do
    the GPU entry points -- both modes run the 32-bit kernel and must equal the literal rule under that table,
    on the sample novel, on a batch large enough for the sliced host path, and in the device-resident call."""
    import torch
    from oracle.loader import Oracle

    path = str(tmp_path / "wide_merges.txt")
    n_merges = wide_merges(merges_path, path, oracle, novel)
    assert n_merges >= 65600
    wide = Oracle(path)
    t = lib.Tokenizer(path, 2048, 50, device=0)
    info = t.table_info()
    assert info["num_merges"] == n_merges and info["max_rank"] >= 65534
    want, woff = wide.encode_fixed(novel, 2048, mode=MODE_GREEDY, threads=NCPU)
    assert want.max() > 65535                              # the new merges really fire
    for m in (lib.GTK_MODE_OPT, lib.GTK_MODE_BASE):
        ids, _, coff, _ = t.encode(novel, mode=m)
        check_chunks(ids, coff, want, woff, f"wide table, novel, mode {m}")
    assert t.decode(ids) == novel
    for piece in (novel[:300], b"", b"a"):                 # tiny batches take the same kernel
        ids, _, coff, _ = t.encode(piece)
        w2, _ = wide.encode_fixed(piece, 2048, mode=MODE_GREEDY)
        assert np.array_equal(ids, w2)
    # 26 MiB: the sliced host path; ragged texts; 32 KiB chunks use the kernel's HBM workspace
    data = np.concatenate([np.frombuffer(novel, np.uint8)] * 4 + [lib.TextGen(3).text(23 << 20, mix=lib.MIX_STRESS)])
    toff = np.array([0, 1000, 1000, len(novel) * 4 + 77, len(data)], dtype=np.int64)
    t32 = lib.Tokenizer(path, 32768, 50, device=0)
    chunk_off = [0]
    for s0, e0 in zip(toff[:-1], toff[1:]):
        chunk_off.extend(list(range(int(s0) + 32768, int(e0), 32768)) + ([int(e0)] if e0 > s0 else []))
    want, woff = wide.encode_chunks(data, np.array(chunk_off, np.int64), mode=MODE_SEGMENTED, threads=NCPU)
    ids, toff_out, coff, _ = t32.encode(data, toff)
    check_chunks(ids, coff, want, woff, "wide table, sliced batch")
    assert toff_out[2] == toff_out[1] and toff_out[-1] == len(ids)
    d_bytes = torch.from_numpy(data[:4 << 20].copy()).cuda()
    d_toff = torch.tensor([0, 4 << 20], dtype=torch.int64, device="cuda")
    d_ids = torch.empty(4 << 20, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    n_ids, n_chunks, _ = t32.encode_device(d_bytes.data_ptr(), 4 << 20, d_toff.data_ptr(), 1, d_ids.data_ptr(), 4 << 20)
    w3, _ = wide.encode_fixed(data[:4 << 20], 32768, mode=MODE_SEGMENTED, threads=NCPU)
    assert n_ids == len(w3) and np.array_equal(d_ids[:n_ids].cpu().numpy(), w3)
    for call in (lambda: t.encode(novel, mode=lib.GTK_MODE_LOCALMIN),
                 lambda: t.encode_chunks_noalloc(d_bytes.data_ptr(), 4096, d_toff.data_ptr(), 1, 4096, d_ids.data_ptr(),
                                                 d_ids.data_ptr())):
        with pytest.raises(lib.GtkError) as e:
            call()
        assert e.value.code == 5
