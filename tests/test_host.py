"""Host-side logic: the C ABI loads and exports what include/gputok_b200.h declares, the table
builder, the host reference entry point, error behaviour, the Python surface, the text
generator and the shard planner (including a 2-rank gloo run).  No GPU needed."""
from __future__ import annotations

import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from conftest import GOLDEN, PKG, ROOT, first_mismatch, fixed_chunk_offsets
from oracle.loader import MODE_GREEDY, MODE_LOCALMIN, MODE_SEGMENTED


def test_library_exports_every_declared_symbol(native_built):
    header = open(os.path.join(ROOT, "include", "gputok_b200.h")).read()
    declared = set(re.findall(r"GTK_API\s+[\w\s\*]+?\b(gtk_\w+)\s*\(", header))
    assert len(declared) >= 17
    lib = ctypes.CDLL(native_built.LIB)
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing
    lib.gtk_version.restype = ctypes.c_char_p
    assert b"sm_100a" in lib.gtk_version()


def test_table_info(native_built, merges_path):
    from gputok_b200 import Tokenizer

    t = Tokenizer(merges_path, 2048, 50, device=-1)
    ti = t.table_info()
    assert ti["vocab_size"] == 50256 and ti["num_merges"] == 50000 and ti["max_rank"] == 49999
    assert ti["monotone"] == 1 and ti["merged_is_256_plus_rank"] == 1 and ti["byte_ids_identity"] == 1
    assert ti["adj_bigrams"] == 2689
    # 65 536 buckets of four 32-bit entries (1 MiB, L2-resident) plus a few overflow pairs
    assert ti["hash_capacity"] == 262144 and 1024 * 1024 <= ti["hash_bytes"] < 1024 * 1024 + 65536
    assert ti["hash_overflow_entries"] < 500 and ti["whole_segment_dropped"] == 0
    assert ti["device"] == -1


def test_crowded_pair_bucket_on_the_host(native_built, merges_path, tmp_path):
    """Pairs beyond the fourth of a bucket live in the side table; the host rule does not care."""
    from conftest import crowded_bucket_merges
    from gputok_b200 import Tokenizer
    from oracle.loader import Oracle

    path = str(tmp_path / "crowded_merges.txt")
    text, n_second = crowded_bucket_merges(merges_path, path)
    t = Tokenizer(path, 512, 50, device=-1)
    ti = t.table_info()
    assert ti["num_merges"] == 1024 + n_second and ti["hash_overflow_entries"] >= n_second - 4 >= 2
    ids, _, coff = t.encode_cpu(np.frombuffer(text, np.uint8))
    want, woff = Oracle(path).encode_fixed(np.frombuffer(text, np.uint8), 512)
    assert np.array_equal(coff, woff) and np.array_equal(ids, want)
    assert (want >= 1280).sum() > 100  # second-level merges do happen in this text


def test_irregular_table_on_the_host(native_built, merges_path, novel, tmp_path):
    from conftest import irregular_merges
    from gputok_b200 import Tokenizer
    from oracle.loader import Oracle

    path = str(tmp_path / "irregular_merges.txt")
    irregular_merges(merges_path, path)
    t = Tokenizer(path, 1000, 50, device=-1)
    ti = t.table_info()
    assert ti["monotone"] == 0 and ti["merged_is_256_plus_rank"] == 0 and ti["byte_ids_identity"] == 1
    data = np.frombuffer(novel[:200_000], np.uint8)
    ids, _, coff = t.encode_cpu(data)
    want, woff = Oracle(path).encode_fixed(data, 1000, threads=os.cpu_count() or 1)
    assert np.array_equal(coff, woff) and np.array_equal(ids, want)


def test_constructor_errors(native_built, merges_path, tmp_path):
    from gputok_b200 import GtkError, Tokenizer

    with pytest.raises(ValueError):
        Tokenizer(merges_path, 0, 50, device=-1)          # std::invalid_argument in the reference
    with pytest.raises(GtkError) as e:
        Tokenizer(str(tmp_path / "nope.txt"), 2048, 50, device=-1)
    assert e.value.code == 2 and "Failed to open merges file" in str(e.value)
    empty = tmp_path / "empty.txt"
    empty.write_bytes(b"")
    with pytest.raises(GtkError) as e:
        Tokenizer(str(empty), 2048, 50, device=-1)
    assert "Empty merges file" in str(e.value)
    t = Tokenizer(merges_path, 16, -3, device=-1)         # max_iters <= 0 -> 50
    assert t.table_info()["max_iters"] == 50


def test_no_cpu_fallback_on_host_only_handle(native_built, merges_path):
    from gputok_b200 import GtkError, Tokenizer

    t = Tokenizer(merges_path, 2048, 50, device=-1)
    with pytest.raises(GtkError) as e:
        t.encode(b"hello world")
    assert e.value.code == 6


def test_malformed_merges_are_parsed_like_the_reference(native_built, oracle, tmp_path):
    """Header skipped, blank and one-field lines consume no rank, duplicate pairs keep the first
    rank, unknown parts become new ids, CRLF tolerated."""
    from gputok_b200 import Tokenizer
    from oracle.loader import Oracle

    p = tmp_path / "m.txt"
    p.write_bytes("#version\nh e\n\nonlyone\nhe l\r\nh e\nl l\nxyz q\nhel l  extra\n".encode())
    t, o = Tokenizer(str(p), 8, 50, device=-1), Oracle(str(p))
    ti = t.table_info()
    assert ti["num_merges"] == o.num_pairs == 5 and ti["vocab_size"] == o.vocab_size
    assert ti["max_rank"] == 5  # six two-field lines, the duplicate consumed rank 2
    data = b"hello hell help xyzq hellhell"
    ids, _, _ = t.encode_cpu(data)
    want, _ = o.encode_fixed(data, 8, mode=MODE_GREEDY)
    assert np.array_equal(ids, want), first_mismatch(ids, want)


def test_host_reference_entry_point_matches_oracle(native_built, merges_path, oracle, novel, ref_cases):
    from gputok_b200 import GTK_RULE_LOCALMIN, Tokenizer

    t = Tokenizer(merges_path, 1024, 50, device=-1)
    data = novel[:120_000]
    ids, toff, coff = t.encode_cpu(data)
    want, woff = oracle.encode_fixed(data, 1024, mode=MODE_GREEDY, threads=os.cpu_count())
    assert np.array_equal(coff, woff) and np.array_equal(ids, want), first_mismatch(ids, want)
    assert toff.tolist() == [0, len(ids)]
    assert t.decode(ids) == data
    # several texts, some empty; adversarial strings recorded from the reference
    blob, case_off = ref_cases["bytes"], ref_cases["case_offsets"]
    ids, toff, coff = t.encode_cpu(blob, case_off)
    want, woff = oracle.encode_chunks(blob, _rechunk(case_off, 1024), mode=MODE_GREEDY)
    assert np.array_equal(ids, want), first_mismatch(ids, want)
    assert np.array_equal(coff, woff)
    # the reference method's own rule (whole text, 50 passes)
    ids, toff, _ = t.encode_cpu(blob, case_off, rule=GTK_RULE_LOCALMIN)
    assert np.array_equal(ids, ref_cases["localmin_ids"])
    assert np.array_equal(toff, ref_cases["localmin_offsets"])


def _rechunk(text_off, chunk):
    out = [0]
    for s, e in zip(text_off[:-1], text_off[1:]):
        out.extend(list(range(int(s) + chunk, int(e), chunk)) + ([int(e)] if e > s else []))
    return np.array(out, dtype=np.int64)


def test_host_greedy_on_generated_strings(native_built, merges_path, oracle):
    """Property test: the host reference entry point (segment cuts + cached ranks) equals the literal
    Algorithm 1 loop on adversarial byte strings -- runs, tiny alphabets, arbitrary bytes, chunk cuts
    inside UTF-8 sequences."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    from gputok_b200 import Tokenizer

    toks = {c: Tokenizer(merges_path, c, 50, device=-1) for c in (1, 3, 16, 4096)}
    piece = st.one_of(
        st.binary(min_size=0, max_size=40),
        st.builds(lambda ch, k: bytes([ch]) * k, st.sampled_from(list(b"ae l\n0.")), st.integers(1, 80)),
        st.text(alphabet="abeilnorst THE,.!\n", min_size=0, max_size=60).map(str.encode),
        st.text(alphabet="\u00e9\u65e5\u672c\U0001F600 a", min_size=0, max_size=20).map(lambda x: x.encode("utf-8")),
    )

    @settings(max_examples=150, deadline=None)
    @given(st.lists(piece, min_size=0, max_size=6), st.sampled_from([1, 3, 16, 4096]))
    def check(pieces, chunk):
        data = b"".join(pieces)
        ids, toff, coff = toks[chunk].encode_cpu(data)
        want, woff = oracle.encode_fixed(data, chunk, mode=MODE_GREEDY)
        assert np.array_equal(ids, want) and np.array_equal(coff, woff)
        assert toks[chunk].decode(ids) == data

    check()


def test_pybind_surface(native_built, merges_path, oracle):
    """Same class and method names as the reference's module (gputok_binding.cu:1015-1065)."""
    import gputok_gpu

    with pytest.raises(ValueError):
        gputok_gpu.GpuTokenizer(merges_path, 0, 50, -1)
    with pytest.raises(RuntimeError):
        gputok_gpu.GpuTokenizer("/nonexistent/merges.txt", 2048, 50, -1)
    tok = gputok_gpu.GpuTokenizer(merges_path, chunk_tokens=2048, max_iters=50, device=-1)
    for name in ("tokenize_batch", "tokenize_batch_blockbpe_base", "tokenize_batch_cpu", "encode_packed"):
        assert hasattr(tok, name)
    texts = ["Hello world!", "", "The weather today is", "naïve café 日本"]
    out = tok.tokenize_batch_cpu(texts)
    assert isinstance(out, list) and len(out) == 4 and out[1] == []
    for text, ids in zip(texts, out):
        raw = text.encode("utf-8")
        want, _ = oracle.encode_fixed(raw, 2048, mode=MODE_GREEDY)
        assert ids == want.tolist()
        assert tok.decode(ids) == raw
    assert tok.tokenize_batch_cpu([]) == []
    lm = tok.tokenize_batch_cpu(texts, merge_rule="localmin")
    want, _ = oracle.encode_chunks(texts[2].encode(), np.array([0, len(texts[2])]), mode=MODE_LOCALMIN)
    assert lm[2] == want.tolist()
    with pytest.raises(RuntimeError):  # GPU entry point on a host-only handle: an error, not a fallback
        tok.tokenize_batch(texts)
    assert tok.table_info()["vocab_size"] == 50256


def test_token_string_writer_reproduces_the_reference_output_file(native_built, merges_path, novel, tmp_path):
    """gtk_write_token_strings == the writer of the standalone binary (gputok_blockbpe.cu:841-865): the file it
    writes for the sample novel at 2048-byte chunks has the sha256 of the reference's committed
    data/output/gpu_tokens_blockbpe.txt (recorded in tests/golden/MANIFEST.json)."""
    import hashlib
    import json

    from gputok_b200 import Tokenizer

    t = Tokenizer(merges_path, 2048, 50, device=-1)
    ids, _, coff = t.encode_cpu(novel)
    out = tmp_path / "gpu_tokens_blockbpe.txt"
    t.write_token_strings(str(out), ids, coff)
    want = json.load(open(os.path.join(GOLDEN, "MANIFEST.json")))["sources"]["data/output/gpu_tokens_blockbpe.txt"]
    assert hashlib.sha256(out.read_bytes()).hexdigest() == want
    assert out.read_bytes().count(b"\n") == 348


def test_textgen_is_deterministic_and_shaped(native_built):
    from gputok_b200 import MIX_STRESS, TextGen

    a = TextGen(1).text(300_000)
    b = TextGen(1).blocks(2, 65536, first_block=1)
    assert np.array_equal(a[65536:3 * 65536], b)          # any block range reproduces the same bytes
    assert np.array_equal(TextGen(1).text(300_000, threads=1), a)
    assert not np.array_equal(TextGen(2).text(4096), a[:4096])
    assert a.max() < 128                                  # plain mix is ASCII
    words = a.tobytes().split()
    assert 3.0 < np.mean([len(w) for w in words]) < 8.0
    s = TextGen(3).text(1 << 20, mix=MIX_STRESS)
    assert (s >= 128).mean() > 0.05                       # multi-byte words present
    runs = re.findall(rb"([a-z ])\1{7,}", s.tobytes())
    assert len(runs) > 50                                 # repeated-byte runs present
    off = TextGen.lognormal_offsets(4, 1 << 22)
    lens = np.diff(off)
    assert off[0] == 0 and off[-1] == 1 << 22 and lens[:-1].min() >= 64 and lens.max() <= 65536
    assert 1500 < np.median(lens) < 2700


def test_shard_planner():
    from gputok_b200.shards import imbalance, partition_by_bytes, split_single_text, stitch_offsets

    rng = np.random.default_rng(0)
    lens = rng.integers(0, 5000, size=1000)
    off = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    for n in (1, 2, 4, 8):
        b = partition_by_bytes(off, n)
        assert b[0] == 0 and b[-1] == 1000 and np.all(np.diff(b) >= 0)
        sizes = [off[b[s + 1]] - off[b[s]] for s in range(n)]
        assert imbalance(sizes) < 1.02
    b = split_single_text(10 * 4096 + 5, 4096, 4)
    assert b[0] == 0 and b[-1] == 10 * 4096 + 5 and all(x % 4096 == 0 for x in b[:-1])
    st = stitch_offsets([np.array([0, 3, 5]), np.array([0, 2]), np.array([0]), np.array([0, 1, 4])])
    assert st.tolist() == [0, 3, 5, 7, 8, 11]
    assert partition_by_bytes(np.array([0]), 4).tolist() == [0, 0, 0, 0, 0]


_GLOO_WORKER = r"""
import os, sys
import numpy as np
import torch.distributed as dist
sys.path[:0] = [{root!r}, {pkg!r}]
from gputok_b200 import TextGen
from gputok_b200.shards import split_single_text, stitch_offsets
from oracle.loader import Oracle, MODE_SEGMENTED

dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
rank, world = dist.get_rank(), dist.get_world_size()
total, chunk = 512 * 1024, 4096
bounds = split_single_text(total, chunk, world)
lo, hi = int(bounds[rank]), int(bounds[rank + 1])
# every rank generates only its own byte range (block-addressable generator)
blk = 65536
mine = TextGen(1).blocks((hi - lo) // blk, blk, first_block=lo // blk)
orc = Oracle({merges!r})
off = np.arange(0, len(mine) + 1, chunk, dtype=np.int64)
ids, ioff = orc.encode_chunks(mine, off, mode=MODE_SEGMENTED)   # stands in for the per-GPU encode
gathered = [None] * world
dist.all_gather_object(gathered, (ids, ioff))                   # test-only: collect to compare
if rank == 0:
    whole = TextGen(1).text(total)
    want, woff = orc.encode_chunks(whole, np.arange(0, total + 1, chunk, dtype=np.int64), mode=MODE_SEGMENTED)
    got = np.concatenate([g[0] for g in gathered])
    goff = stitch_offsets([g[1] for g in gathered])
    assert np.array_equal(got, want) and np.array_equal(goff, woff)
    print("SHARDS_OK", len(got))
dist.barrier()
dist.destroy_process_group()
"""


def test_two_rank_sharding_over_gloo(native_built, merges_path, oracle, tmp_path):
    """The N>1 path on CPU: byte-range shards, independent encodes, host-side offset stitching."""
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER.format(root=ROOT, pkg=PKG, port=port, merges=merges_path))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                              text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "SHARDS_OK" in outs[0]


def test_host_table_beyond_16_bits(native_built, merges_path, oracle, novel, tmp_path):
    """A merges file with more than 65 534 merges builds (the reference accepts any file); the host tokenizer
    equals the oracle under that table and the new, high ids really occur."""
    import gputok_b200
    from conftest import wide_merges
    from oracle.loader import MODE_GREEDY, Oracle

    path = str(tmp_path / "wide_merges.txt")
    n = wide_merges(merges_path, path, oracle, novel[:200000], extra=16000)
    assert n > 65534
    tok = gputok_b200.Tokenizer(path, 1024, 50, device=-1)
    assert tok.table_info()["num_merges"] == n
    part = novel[:60000]
    ids, _, coff = tok.encode_cpu(part)
    want, woff = Oracle(path).encode_fixed(part, 1024, mode=MODE_GREEDY, threads=4)
    assert np.array_equal(ids, want) and np.array_equal(coff, woff)
    assert ids.max() > 65535


def test_bench_reference_arm_line(native_built, oracle):
    """`bench.py --impl reference` needs no GPU: it prints one JSON line with the contract's keys, describes the
    same workload as the GPU arm would, and reports zero copy bytes."""
    import json

    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--ref-budget-s", "1", "--bytes", str(8 << 20)],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "input_MB_per_s" and d["unit"] == "MB/s" and d["value"] > 0
    assert d["config"]["workload"] == "cfg2" and d["config"]["chunk_bytes"] == 4096 and d["config"]["bytes_per_gpu"] == 8 << 20
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0 and d["higher_is_better"] is True
