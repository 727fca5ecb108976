"""ctypes loaders for the parity checkers.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by the CPU-baseline legs of ``bench.py``.  The tokenizer package never
imports this module.

``Oracle``  wraps ``_build/libbpe_oracle.so`` (the plain-C restatement,
``bpe_oracle.c``); ``RefGreedy`` wraps ``_ref/libref_greedy.so`` (the
reference's own host functions compiled in place by the Makefile; only
available where that file was built).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libbpe_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libref_greedy.so")

MODE_GREEDY = 0      # literal Algorithm 1 (bpe_merge_cpu_greedy)
MODE_SEGMENTED = 1   # literal Algorithm 1 on never-merge segments (oracle only)
MODE_LOCALMIN = 2    # the binding's bpe_merge_cpu rule (not the parity target)


def reference_root() -> str:
    """Where the reference checkout is expected: ``$GTK_REFERENCE_ROOT``, else a directory named
    ``reference`` beside the repository.  It need not exist (the GPU box has none)."""
    return os.environ.get("GTK_REFERENCE_ROOT") or os.path.abspath(os.path.join(HERE, "..", "..", "reference"))


def build(ref: bool | None = None) -> None:
    """Compile the checkers (gcc/g++ only).  ``ref=None``: also compile the reference's own host
    functions when its checkout is present."""
    if ref is None:
        ref = os.path.isfile(os.path.join(reference_root(), "gputok_blockbpe.cu"))
    targets = ["oracle"] + (["ref"] if ref else [])
    subprocess.run(["make", "-s", "-C", HERE, "REF_ROOT=" + reference_root()] + targets, check=True)


def _u8(a) -> np.ndarray:
    if isinstance(a, (bytes, bytearray, memoryview)):
        return np.frombuffer(a, dtype=np.uint8)
    return np.ascontiguousarray(a, dtype=np.uint8)


class _Chunked:
    """Shared driver for the two libraries' ``*_encode_chunks`` entry points."""

    _encode = None
    _h = None

    def encode_chunks(self, data, chunk_off, mode: int = MODE_GREEDY, max_iters: int = 50,
                      threads: int = 1):
        """Tokenise ``data[chunk_off[c]:chunk_off[c+1]]`` for every c.

        Returns ``(ids int32[total], offsets int64[C+1])``.
        """
        buf = _u8(data)
        off = np.ascontiguousarray(chunk_off, dtype=np.int64)
        n_chunks = len(off) - 1
        if n_chunks <= 0:
            return np.zeros(0, np.int32), np.zeros(1, np.int64)
        span = int(off[-1] - off[0])
        ids = np.empty(max(span, 1), dtype=np.int32)
        out_off = np.empty(n_chunks + 1, dtype=np.int64)
        total = self._encode(self._h, buf.ctypes.data_as(C.c_void_p), off.ctypes.data_as(C.c_void_p),
                             C.c_int64(n_chunks), ids.ctypes.data_as(C.c_void_p),
                             out_off.ctypes.data_as(C.c_void_p), int(mode), int(max_iters), int(threads))
        return ids[:total].copy(), out_off

    def encode_fixed(self, data, chunk_bytes: int, **kw):
        """Fixed-size chunking of one text, as the reference's chunk loop does
        (gputok_blockbpe.cu:621-632)."""
        n = len(_u8(data))
        off = np.arange(0, n + chunk_bytes, chunk_bytes, dtype=np.int64)
        off = off[off < n]
        off = np.append(off, n).astype(np.int64) if n else np.zeros(1, np.int64)
        return self.encode_chunks(data, off, **kw)


class Oracle(_Chunked):
    def __init__(self, merges_path: str):
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        lib = C.CDLL(ORACLE_SO)
        lib.bpe_oracle_create.restype = C.c_void_p
        lib.bpe_oracle_create.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        lib.bpe_oracle_destroy.argtypes = [C.c_void_p]
        lib.bpe_oracle_vocab_size.restype = C.c_int32
        lib.bpe_oracle_vocab_size.argtypes = [C.c_void_p]
        lib.bpe_oracle_num_pairs.restype = C.c_int64
        lib.bpe_oracle_num_pairs.argtypes = [C.c_void_p]
        lib.bpe_oracle_byte_id.restype = C.c_int32
        lib.bpe_oracle_byte_id.argtypes = [C.c_void_p, C.c_int]
        lib.bpe_oracle_dump_pairs.restype = C.c_int64
        lib.bpe_oracle_dump_pairs.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        lib.bpe_oracle_token_symbols.restype = C.c_int32
        lib.bpe_oracle_token_symbols.argtypes = [C.c_void_p, C.c_int32, C.c_char_p, C.c_int32]
        lib.bpe_oracle_token_id.restype = C.c_int32
        lib.bpe_oracle_token_id.argtypes = [C.c_void_p, C.c_char_p, C.c_int32]
        lib.bpe_oracle_token_bytes.restype = C.c_int32
        lib.bpe_oracle_token_bytes.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32]
        lib.bpe_oracle_decode.restype = C.c_int64
        lib.bpe_oracle_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64]
        lib.bpe_oracle_adj_bitmap.argtypes = [C.c_void_p, C.c_void_p]
        lib.bpe_oracle_greedy.restype = C.c_int64
        lib.bpe_oracle_greedy.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        lib.bpe_oracle_encode_chunks.restype = C.c_int64
        lib.bpe_oracle_encode_chunks.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                                 C.c_void_p, C.c_int, C.c_int, C.c_int]
        self.lib = lib
        err = C.create_string_buffer(512)
        self._h = lib.bpe_oracle_create(merges_path.encode(), err, 512)
        if not self._h:
            raise RuntimeError(err.value.decode() or "bpe_oracle_create failed")
        self._encode = lib.bpe_oracle_encode_chunks

    def __del__(self):
        if getattr(self, "_h", None):
            self.lib.bpe_oracle_destroy(self._h)
            self._h = None

    @property
    def vocab_size(self) -> int:
        return self.lib.bpe_oracle_vocab_size(self._h)

    @property
    def num_pairs(self) -> int:
        return self.lib.bpe_oracle_num_pairs(self._h)

    def byte_id(self, b: int) -> int:
        return self.lib.bpe_oracle_byte_id(self._h, b)

    def pairs(self) -> np.ndarray:
        """All merges as rows (left, right, rank, merged), sorted by rank."""
        rows = np.empty((self.num_pairs, 4), dtype=np.int32)
        n = self.lib.bpe_oracle_dump_pairs(self._h, rows.ctypes.data_as(C.c_void_p), len(rows))
        rows = rows[:n]
        return rows[np.argsort(rows[:, 2], kind="stable")]

    def token_symbols(self, tid: int) -> bytes:
        buf = C.create_string_buffer(4096)
        n = self.lib.bpe_oracle_token_symbols(self._h, tid, buf, 4096)
        if n < 0:
            raise KeyError(tid)
        return buf.raw[:n]

    def token_id(self, symbols: bytes) -> int:
        return self.lib.bpe_oracle_token_id(self._h, symbols, len(symbols))

    def token_bytes(self, tid: int) -> bytes:
        buf = (C.c_uint8 * 4096)()
        n = self.lib.bpe_oracle_token_bytes(self._h, tid, buf, 4096)
        if n < 0:
            raise KeyError(tid)
        return bytes(buf[:n])

    def decode(self, ids) -> bytes:
        a = np.ascontiguousarray(ids, dtype=np.int32)
        cap = 64 * max(len(a), 1)
        out = np.empty(cap, dtype=np.uint8)
        n = self.lib.bpe_oracle_decode(self._h, a.ctypes.data_as(C.c_void_p), len(a),
                                       out.ctypes.data_as(C.c_void_p), cap)
        if n < 0:
            raise ValueError("undecodable id or overflow")
        return out[:n].tobytes()

    def adj_bitmap(self) -> np.ndarray:
        out = np.zeros(2048, dtype=np.uint32)
        self.lib.bpe_oracle_adj_bitmap(self._h, out.ctypes.data_as(C.c_void_p))
        return out

    def greedy_ids(self, ids) -> np.ndarray:
        """Literal Algorithm 1 on one id sequence."""
        a = np.array(ids, dtype=np.int32)
        n = self.lib.bpe_oracle_greedy(self._h, a.ctypes.data_as(C.c_void_p), len(a))
        return a[:n].copy()


class RefGreedy(_Chunked):
    """The reference's own bpe_merge_cpu_greedy / bpe_merge_cpu (compiled in place)."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self, merges_path: str):
        lib = C.CDLL(REF_SO)
        lib.ref_create.restype = C.c_void_p
        lib.ref_create.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        lib.ref_destroy.argtypes = [C.c_void_p]
        lib.ref_vocab_size.restype = C.c_int32
        lib.ref_vocab_size.argtypes = [C.c_void_p]
        lib.ref_num_pairs.restype = C.c_int64
        lib.ref_num_pairs.argtypes = [C.c_void_p]
        lib.ref_dump_pairs.restype = C.c_int64
        lib.ref_dump_pairs.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
        lib.ref_token_symbols.restype = C.c_int32
        lib.ref_token_symbols.argtypes = [C.c_void_p, C.c_int32, C.c_char_p, C.c_int32]
        lib.ref_encode_chunks.restype = C.c_int64
        lib.ref_encode_chunks.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                          C.c_void_p, C.c_int, C.c_int, C.c_int]
        self.lib = lib
        err = C.create_string_buffer(512)
        self._h = lib.ref_create(merges_path.encode(), err, 512)
        if not self._h:
            raise RuntimeError(err.value.decode() or "ref_create failed")
        self._encode = lib.ref_encode_chunks

    def __del__(self):
        if getattr(self, "_h", None):
            self.lib.ref_destroy(self._h)
            self._h = None

    @property
    def vocab_size(self) -> int:
        return self.lib.ref_vocab_size(self._h)

    @property
    def num_pairs(self) -> int:
        return self.lib.ref_num_pairs(self._h)

    def pairs(self) -> np.ndarray:
        rows = np.empty((self.num_pairs, 4), dtype=np.int32)
        n = self.lib.ref_dump_pairs(self._h, rows.ctypes.data_as(C.c_void_p), len(rows))
        rows = rows[:n]
        return rows[np.argsort(rows[:, 2], kind="stable")]

    def token_symbols(self, tid: int) -> bytes:
        buf = C.create_string_buffer(4096)
        n = self.lib.ref_token_symbols(self._h, tid, buf, 4096)
        if n < 0:
            raise KeyError(tid)
        return buf.raw[:n]
