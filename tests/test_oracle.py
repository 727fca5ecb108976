"""The CPU oracle (oracle/bpe_oracle.c) against the reference's own golden vectors and host
functions.  These pins are what makes the GPU parity tests meaningful."""
from __future__ import annotations

import os

import numpy as np
import pytest

from conftest import first_mismatch, fixed_chunk_offsets
from oracle.loader import MODE_GREEDY, MODE_LOCALMIN, MODE_SEGMENTED, RefGreedy


def test_table_matches_reference_properties(oracle):
    # values measured from the reference's build_vocab_and_merges (gputok_blockbpe.cu:178-236)
    assert oracle.vocab_size == 50256
    assert oracle.num_pairs == 50000
    assert all(oracle.byte_id(b) == b for b in range(256))
    rows = oracle.pairs()
    assert np.array_equal(rows[:, 2], np.arange(50000))
    assert np.array_equal(rows[:, 3], rows[:, 2] + 256)
    # first merges of GPT-2: "Ġ t", "Ġ a", "h e"
    assert rows[0, :2].tolist() == [0x20, ord("t")] and rows[2, :2].tolist() == [ord("h"), ord("e")]
    assert int(sum(bin(int(w)).count("1") for w in oracle.adj_bitmap())) == 2689


def test_golden_blockbpe_output(oracle, novel, golden_2048):
    """data/output/gpu_tokens_blockbpe.txt == literal greedy on the sample novel at 2048-byte chunks."""
    gold_ids, gold_off = golden_2048
    ids, off = oracle.encode_fixed(novel, 2048, mode=MODE_GREEDY, threads=os.cpu_count())
    assert len(off) == len(gold_off) == 349
    assert np.array_equal(off, gold_off), first_mismatch(off, gold_off)
    assert np.array_equal(ids, gold_ids), first_mismatch(ids, gold_ids)
    assert oracle.decode(ids) == novel


def test_reference_host_function_outputs(oracle, ref_cases):
    """Adversarial strings: outputs recorded from the reference's bpe_merge_cpu_greedy / bpe_merge_cpu."""
    data, coff = ref_cases["bytes"], ref_cases["case_offsets"]
    ids, off = oracle.encode_chunks(data, coff, mode=MODE_GREEDY)
    assert np.array_equal(off, ref_cases["greedy_offsets"])
    assert np.array_equal(ids, ref_cases["greedy_ids"])
    ids, off = oracle.encode_chunks(data, coff, mode=MODE_SEGMENTED)
    assert np.array_equal(off, ref_cases["greedy_offsets"])
    assert np.array_equal(ids, ref_cases["greedy_ids"])
    ids, off = oracle.encode_chunks(data, coff, mode=MODE_LOCALMIN, max_iters=50)
    assert np.array_equal(off, ref_cases["localmin_offsets"])
    assert np.array_equal(ids, ref_cases["localmin_ids"])


def test_localmin_golden_is_not_greedy(oracle):
    """data/output/gpu_tokens_optimized.txt follows the binding's local-minimum rule, not Algorithm 1."""
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_localmin_512.npz"))
    text, gold = z["text"], z["ids"]
    lm, _ = oracle.encode_chunks(text, np.array([0, len(text)]), mode=MODE_LOCALMIN, max_iters=50)
    gr, _ = oracle.encode_chunks(text, np.array([0, len(text)]), mode=MODE_GREEDY)
    assert np.array_equal(lm, gold)
    assert len(gr) < len(gold) and not np.array_equal(gr, gold[:len(gr)])


@pytest.mark.parametrize("chunk", [1, 2, 3, 7, 64, 512, 1024, 4096])
def test_segmented_equals_literal_on_novel(oracle, novel, chunk):
    data = novel[:200_000] if chunk >= 64 else novel[:20_000]
    a, ao = oracle.encode_fixed(data, chunk, mode=MODE_GREEDY, threads=os.cpu_count())
    b, bo = oracle.encode_fixed(data, chunk, mode=MODE_SEGMENTED, threads=os.cpu_count())
    assert np.array_equal(ao, bo) and np.array_equal(a, b), first_mismatch(a, b)


def test_segmented_equals_literal_on_stress_text(oracle, native_built):
    from gputok_b200 import MIX_STRESS, TextGen

    data = TextGen(3).text(256 * 1024, mix=MIX_STRESS)
    off = fixed_chunk_offsets(len(data), 32768)
    a, ao = oracle.encode_chunks(data, off, mode=MODE_GREEDY, threads=os.cpu_count())
    b, bo = oracle.encode_chunks(data, off, mode=MODE_SEGMENTED, threads=os.cpu_count())
    assert np.array_equal(ao, bo) and np.array_equal(a, b), first_mismatch(a, b)
    assert oracle.decode(a) == data.tobytes()


def test_single_sequence_api(oracle):
    # "the" -> th + e -> the ; ids are 256 + rank
    out = oracle.greedy_ids([ord(c) for c in " the"])
    assert len(out) == 1 and oracle.token_bytes(int(out[0])) == b" the"
    assert oracle.greedy_ids([]).size == 0
    assert oracle.greedy_ids([65]).tolist() == [65]


@pytest.mark.skipif(not RefGreedy.available(), reason="reference host functions not compiled here")
def test_against_live_reference_functions(oracle, merges_path, novel, native_built):
    """Where oracle/_ref was built: compare with the reference's functions directly."""
    from gputok_b200 import MIX_STRESS, TextGen

    ref = RefGreedy(merges_path)
    assert ref.vocab_size == oracle.vocab_size and np.array_equal(ref.pairs(), oracle.pairs())
    for tid in (0, 32, 255, 256, 1000, 50255):
        assert ref.token_symbols(tid) == oracle.token_symbols(tid)
    for data, chunk in ((novel[:150_000], 1024), (TextGen(0).text(128 * 1024).tobytes(), 1024),
                        (TextGen(3).text(64 * 1024, mix=MIX_STRESS).tobytes(), 4096)):
        off = fixed_chunk_offsets(len(data), chunk)
        a, ao = ref.encode_chunks(data, off, mode=MODE_GREEDY, threads=os.cpu_count())
        b, bo = oracle.encode_chunks(data, off, mode=MODE_GREEDY, threads=os.cpu_count())
        assert np.array_equal(ao, bo) and np.array_equal(a, b), first_mismatch(a, b)
        a, ao = ref.encode_chunks(data, off, mode=MODE_LOCALMIN, max_iters=50, threads=os.cpu_count())
        b, bo = oracle.encode_chunks(data, off, mode=MODE_LOCALMIN, max_iters=50, threads=os.cpu_count())
        assert np.array_equal(ao, bo) and np.array_equal(a, b), first_mismatch(a, b)
