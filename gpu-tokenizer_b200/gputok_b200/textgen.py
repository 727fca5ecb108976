"""ctypes binding of the seeded synthetic text generator (csrc/gtk_textgen.c)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

MIX_PLAIN = 0   # ASCII words only
MIX_STRESS = 1  # + 20 % multi-byte UTF-8 words, 5 % runs of 8..256 equal bytes

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB = None


def _lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_PKG_ROOT, "libgtk_textgen.so")
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python build.py` in {_PKG_ROOT}")
        lib = C.CDLL(path)
        lib.gtk_textgen_create.restype = C.c_void_p
        lib.gtk_textgen_create.argtypes = [C.c_uint64]
        lib.gtk_textgen_destroy.argtypes = [C.c_void_p]
        lib.gtk_textgen_fill.argtypes = [C.c_void_p, C.c_uint64, C.c_int, C.c_void_p, C.c_int64]
        lib.gtk_textgen_blocks.argtypes = [C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int]
        lib.gtk_textgen_lognormal_offsets.restype = C.c_int64
        lib.gtk_textgen_lognormal_offsets.argtypes = [C.c_uint64, C.c_double, C.c_double, C.c_int64, C.c_int64,
                                                      C.c_int64, C.c_void_p, C.c_int64]
        _LIB = lib
    return _LIB


class TextGen:
    """Deterministic text for one seed.  A text is a sequence of independent blocks of
    ``block_bytes``; any block range can be generated on its own."""

    def __init__(self, seed: int):
        self.seed = int(seed)
        self._h = _lib().gtk_textgen_create(self.seed)
        if not self._h:
            raise MemoryError("gtk_textgen_create")

    def __del__(self):
        if getattr(self, "_h", None):
            _lib().gtk_textgen_destroy(self._h)
            self._h = None

    def blocks(self, n_blocks: int, block_bytes: int = 65536, first_block: int = 0, mix: int = MIX_PLAIN,
               threads: int | None = None, out: np.ndarray | None = None) -> np.ndarray:
        n = int(n_blocks) * int(block_bytes)
        if out is None:
            out = np.empty(n, dtype=np.uint8)
        assert out.dtype == np.uint8 and out.size >= n and out.flags.c_contiguous
        if threads is None:
            threads = min(os.cpu_count() or 1, 64)
        _lib().gtk_textgen_blocks(self._h, int(mix), int(block_bytes), int(first_block), int(n_blocks),
                                  out.ctypes.data, int(threads))
        return out[:n]

    def text(self, n_bytes: int, block_bytes: int = 65536, mix: int = MIX_PLAIN, threads: int | None = None,
             out: np.ndarray | None = None) -> np.ndarray:
        """The first n_bytes of the seed's text (n_bytes need not be a block multiple)."""
        nb = (int(n_bytes) + block_bytes - 1) // block_bytes
        if out is not None and out.size >= nb * block_bytes:
            return self.blocks(nb, block_bytes, 0, mix, threads, out)[:n_bytes]
        return self.blocks(nb, block_bytes, 0, mix, threads)[:n_bytes]

    @staticmethod
    def lognormal_offsets(seed: int, total_bytes: int, median: float = 2048.0, sigma: float = 1.0, lo: int = 64,
                          hi: int = 65536) -> np.ndarray:
        """Offsets of pieces with log-normal lengths (clipped to [lo, hi]) covering total_bytes."""
        cap = int(total_bytes) // int(lo) + 2
        off = np.empty(cap, dtype=np.int64)
        n = _lib().gtk_textgen_lognormal_offsets(int(seed), float(median), float(sigma), int(lo), int(hi),
                                                 int(total_bytes), off.ctypes.data, cap)
        if n < 0:
            raise RuntimeError("offset buffer too small")
        return off[:n + 1].copy()
