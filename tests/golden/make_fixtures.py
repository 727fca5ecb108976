"""Regenerates the committed fixtures from the reference tree (run where it is mounted).

    python tests/golden/make_fixtures.py <reference root>

Writes next to this script:
  gpt2_merges.txt            the reference's data/gpt2_tokenizer/merges.txt (the merge table every
                             configuration uses; data, not code), byte-for-byte
  pride_and_prejudice.txt.gz the reference's sample input data/input/pride_and_prejudice.txt
  golden_blockbpe_2048.npz   ids of the reference's committed output data/output/gpu_tokens_blockbpe.txt
                             (348 chunks of 2048 bytes of the sample input; token strings mapped to ids
                             through the vocabulary rebuilt from merges.txt) + per-chunk offsets
  golden_localmin_512.npz    the 512-byte text and ids of data/output/gpu_tokens_optimized.txt (the
                             reference's OTHER merge rule; pins the localmin switch only)
  ref_greedy_cases.npz       outputs of the reference's own bpe_merge_cpu_greedy (compiled in place by
                             oracle/Makefile) on adversarial byte strings
  MANIFEST.json              sha256 of every source and product
The test-suite reads only these files; the reference tree is not needed at test time.
"""
from __future__ import annotations

import gzip
import hashlib
import json
import os
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def sha(path_or_bytes) -> str:
    data = open(path_or_bytes, "rb").read() if isinstance(path_or_bytes, str) else path_or_bytes
    return hashlib.sha256(data).hexdigest()


def adversarial_cases() -> list[bytes]:
    rng = np.random.default_rng(1234)
    cases = [b"", b"a", b"ab", b"the", b" the", b"aaaa", b"a" * 255, b"a" * 256, b"\n" * 101, b"e" * 77, b"l" * 33,
             b"0" * 50, b" " * 200, b"ab" * 100, b"abc" * 70, b"the the the the", b"Hello world!",
             "日本語のテキスト".encode(), ("😀" * 40).encode(), ("é" * 90).encode(), "naïve café".encode(),
             b"\x00\x01\x02\xff\xfe", bytes(range(256)), b"ing" * 64 + b"tion" * 32,
             b"aaaaaaaaaaaaaaaab" * 20, b"xxxxxxxxyyyyyyyyzzzzzzzz" * 8, b"....!!!!????,,,,", b"1234567890" * 12,
             b"        indented\n\n\n\tcode();\r\n", b"ss" * 40 + b"s", b"eeee ee e eee eeeee eeeeee"]
    for n in (1, 2, 3, 7, 31, 32, 33, 63, 64, 65, 127, 128, 129, 300, 511, 513):
        cases.append(bytes(rng.integers(97, 123, size=n, dtype=np.uint8)))      # random lowercase
        cases.append(bytes(rng.integers(0, 256, size=n, dtype=np.uint8)))       # random bytes
        cases.append(bytes(rng.choice(np.frombuffer(b"aab e", dtype=np.uint8), size=n)))  # tiny alphabet
    return cases


def main() -> None:
    from oracle.loader import MODE_GREEDY, MODE_LOCALMIN, Oracle, RefGreedy, build, reference_root

    ref = sys.argv[1] if len(sys.argv) > 1 else reference_root()
    os.environ["GTK_REFERENCE_ROOT"] = ref

    build(ref=True)
    manifest = {"reference": "venugopalkadamba/gpu-tokenizer", "sources": {}, "products": {}}

    merges_src = os.path.join(ref, "data/gpt2_tokenizer/merges.txt")
    merges_dst = os.path.join(HERE, "gpt2_merges.txt")
    shutil.copyfile(merges_src, merges_dst)
    manifest["sources"]["data/gpt2_tokenizer/merges.txt"] = sha(merges_src)

    pp_src = os.path.join(ref, "data/input/pride_and_prejudice.txt")
    text = open(pp_src, "rb").read()
    with open(os.path.join(HERE, "pride_and_prejudice.txt.gz"), "wb") as f:
        f.write(gzip.compress(text, compresslevel=9, mtime=0))
    manifest["sources"]["data/input/pride_and_prejudice.txt"] = sha(text)

    orc = Oracle(merges_dst)
    golden_src = os.path.join(ref, "data/output/gpu_tokens_blockbpe.txt")
    lines = open(golden_src, "rb").read().split(b"\n")
    assert lines[-1] == b""
    ids, off = [], [0]
    for line in lines[:-1]:
        for sym in line.split(b" "):
            tid = orc.token_id(sym)
            assert tid >= 0, sym
            ids.append(tid)
        off.append(len(ids))
    np.savez_compressed(os.path.join(HERE, "golden_blockbpe_2048.npz"), ids=np.array(ids, np.uint16),
                        offsets=np.array(off, np.int64), chunk_bytes=np.int64(2048))
    manifest["sources"]["data/output/gpu_tokens_blockbpe.txt"] = sha(golden_src)

    lm_src = os.path.join(ref, "data/output/gpu_tokens_optimized.txt")
    syms = open(lm_src, "rb").read().strip().split(b" ")
    lm_ids = np.array([orc.token_id(s) for s in syms], np.int32)
    assert (lm_ids >= 0).all()
    lm_text = orc.decode(lm_ids)
    np.savez_compressed(os.path.join(HERE, "golden_localmin_512.npz"), ids=lm_ids,
                        text=np.frombuffer(lm_text, np.uint8))
    manifest["sources"]["data/output/gpu_tokens_optimized.txt"] = sha(lm_src)

    refg = RefGreedy(merges_dst)
    cases = adversarial_cases()
    blob = b"".join(cases)
    coff = np.zeros(len(cases) + 1, np.int64)
    coff[1:] = np.cumsum([len(c) for c in cases])
    g_ids, g_off = refg.encode_chunks(blob, coff, mode=MODE_GREEDY, threads=4)
    l_ids, l_off = refg.encode_chunks(blob, coff, mode=MODE_LOCALMIN, max_iters=50, threads=4)
    np.savez_compressed(os.path.join(HERE, "ref_greedy_cases.npz"), bytes=np.frombuffer(blob, np.uint8),
                        case_offsets=coff, greedy_ids=g_ids, greedy_offsets=g_off, localmin_ids=l_ids,
                        localmin_offsets=l_off)

    for name in sorted(os.listdir(HERE)):
        if name.endswith((".npz", ".gz", ".txt")):
            manifest["products"][name] = sha(os.path.join(HERE, name))
    with open(os.path.join(HERE, "MANIFEST.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    print(json.dumps(manifest["products"], indent=1))


if __name__ == "__main__":
    main()
