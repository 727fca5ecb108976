"""ctypes binding of include/gputok_b200.h."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

GTK_MODE_OPT = 0
GTK_MODE_BASE = 1
GTK_MODE_LOCALMIN = 2  # the reference's other rule (local minimum, max_iters passes), per chunk
GTK_RULE_GREEDY = 0
GTK_RULE_LOCALMIN = 1
NOALLOC_MAX_CHUNK_BYTES = 16384

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB = None


class GtkError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"gputok_b200 error {code}: {message}")
        self.code = code


class _TableInfo(C.Structure):
    _fields_ = [("vocab_size", C.c_int32), ("num_merges", C.c_int32), ("max_rank", C.c_uint32),
                ("hash_capacity", C.c_uint32), ("hash_overflow_entries", C.c_uint32), ("hash_bytes", C.c_uint32),
                ("monotone", C.c_int32), ("merged_is_256_plus_rank", C.c_int32), ("byte_ids_identity", C.c_int32),
                ("adj_bigrams", C.c_int32), ("chunk_tokens", C.c_int32), ("max_iters", C.c_int32),
                ("device", C.c_int32), ("sm_count", C.c_int32),
                ("whole_segment_entries", C.c_int32), ("whole_segment_dropped", C.c_uint32)]


def library_path() -> str:
    """The CUDA library beside the package; ``GPUTOK_B200_LIBRARY`` names another build of it (the
    bounds-checked one, ``libgputok_b200_checked.so``)."""
    return os.environ.get("GPUTOK_B200_LIBRARY") or os.path.join(_PKG_ROOT, "libgputok_b200.so")


def checked_library_path() -> str:
    return os.path.join(_PKG_ROOT, "libgputok_b200_checked.so")


def load_library() -> C.CDLL:
    """Load the CUDA library.  Raises if it has not been built: there is no other code path."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not os.path.exists(path):
        raise GtkError(-1, f"{path} is missing: run `python build.py` in {_PKG_ROOT} (needs nvcc); "
                           "the tokenizer has no CPU fallback")
    lib = C.CDLL(path)
    vp, i64, i32 = C.c_void_p, C.c_int64, C.c_int32
    lib.gtk_version.restype = C.c_char_p
    lib.gtk_global_error.restype = C.c_char_p
    lib.gtk_create.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.POINTER(vp)]
    lib.gtk_destroy.argtypes = [vp]
    lib.gtk_destroy.restype = None
    lib.gtk_last_error.argtypes = [vp]
    lib.gtk_last_error.restype = C.c_char_p
    lib.gtk_table_info_get.argtypes = [vp, C.POINTER(_TableInfo)]
    lib.gtk_encode.argtypes = [vp, C.c_int, vp, vp, i64, C.POINTER(C.c_float)]
    lib.gtk_encode_cpu.argtypes = [vp, C.c_int, vp, vp, i64]
    lib.gtk_result_sizes.argtypes = [vp, C.POINTER(i64), C.POINTER(i64), C.POINTER(i64)]
    lib.gtk_result_view.argtypes = [vp, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]
    lib.gtk_result_copy.argtypes = [vp, vp, i64, vp, vp, i64]
    lib.gtk_encode_device.argtypes = [vp, C.c_int, vp, i64, vp, i64, vp, i64, vp, i64, C.POINTER(i64),
                                      C.POINTER(i64), C.POINTER(C.c_float)]
    lib.gtk_last_stage_ms.argtypes = [vp, C.POINTER(C.c_float * 5), C.POINTER(i32)]
    lib.gtk_decode.argtypes = [vp, vp, i64, vp, i64, C.POINTER(i64)]
    lib.gtk_token_symbols.argtypes = [vp, i32, C.c_char_p, i32]
    lib.gtk_token_symbols.restype = i32
    lib.gtk_set_stream.argtypes = [vp, vp]
    lib.gtk_set_id_space.argtypes = [vp, C.c_int]
    lib.gtk_set_base_block_size.argtypes = [vp, C.c_int]
    lib.gtk_set_stage_timing.argtypes = [vp, C.c_int]
    lib.gtk_write_token_strings.argtypes = [vp, C.c_char_p, vp, vp, i64]
    lib.gtk_encode_chunks_noalloc.argtypes = [vp, vp, i64, vp, i64, i32, vp, vp]
    lib.gtk_pinned_alloc.argtypes = [C.c_size_t]
    lib.gtk_pinned_alloc.restype = vp
    lib.gtk_pinned_free.argtypes = [vp]
    lib.gtk_pinned_free.restype = None
    _LIB = lib
    return lib


def _as_u8(data) -> np.ndarray:
    if isinstance(data, (bytes, bytearray, memoryview)):
        return np.frombuffer(data, dtype=np.uint8)
    return np.ascontiguousarray(data, dtype=np.uint8)


class PinnedArray:
    """A numpy view over page-locked host memory from gtk_pinned_alloc."""

    def __init__(self, nbytes: int):
        self._lib = load_library()
        self._ptr = self._lib.gtk_pinned_alloc(max(int(nbytes), 1))
        if not self._ptr:
            raise GtkError(-1, "gtk_pinned_alloc failed")
        buf = (C.c_uint8 * max(int(nbytes), 1)).from_address(self._ptr)
        self.array = np.frombuffer(buf, dtype=np.uint8)[:nbytes]

    def free(self) -> None:
        if self._ptr:
            self.array = None
            self._lib.gtk_pinned_free(self._ptr)
            self._ptr = None

    def __del__(self):
        self.free()


class Tokenizer:
    """One handle of the C ABI (one device, one stream).

    ``device=-1`` builds a host-only handle (table + ``encode_cpu``); its GPU
    entry points raise.
    """

    def __init__(self, merges_path: str, chunk_tokens: int = 2048, max_iters: int = 50, device: int = 0):
        self._lib = load_library()
        h = C.c_void_p()
        rc = self._lib.gtk_create(os.fsencode(merges_path), int(chunk_tokens), int(max_iters), int(device),
                                  C.byref(h))
        if rc != 0:
            msg = self._lib.gtk_global_error().decode()
            if rc == 1:
                raise ValueError(msg)
            raise GtkError(rc, msg)
        self._h = h
        self.chunk_tokens = int(chunk_tokens)
        self.device = int(device)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.gtk_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise GtkError(rc, self._lib.gtk_last_error(self._h).decode())

    # ------------------------------------------------------------------ info
    def table_info(self) -> dict:
        ti = _TableInfo()
        self._check(self._lib.gtk_table_info_get(self._h, C.byref(ti)))
        return {name: getattr(ti, name) for name, _ in _TableInfo._fields_}

    def stage_ms(self) -> dict:
        ms = (C.c_float * 5)()
        n = C.c_int32()
        self._check(self._lib.gtk_last_stage_ms(self._h, C.byref(ms), C.byref(n)))
        return {"chunker": ms[0], "merge": ms[1], "scan": ms[2], "pack": ms[3], "pipeline": ms[4],
                "kernel_launches": n.value}

    def set_stream(self, cuda_stream: int | None) -> None:
        """Run later GPU work on the caller's stream (e.g. ``torch.cuda.current_stream().cuda_stream``).

        ``None`` restores the handle's own (non-blocking) stream.  The integer 0 -- what a framework
        reports for the legacy default stream -- selects that stream (passed on as cudaStreamLegacy),
        so work queued there by the caller is ordered before the tokenizer's kernels."""
        if cuda_stream is None:
            ptr = None
        elif int(cuda_stream) == 0:
            ptr = 1  # cudaStreamLegacy
        else:
            ptr = int(cuda_stream)
        self._check(self._lib.gtk_set_stream(self._h, ptr))

    def set_id_space(self, gpt2: bool) -> None:
        """False (default): ids as the reference produces them (ids < 256 are byte values);
        True: ids < 256 remapped to GPT-2's own vocabulary order (feedable to a GPT-2 model)."""
        self._check(self._lib.gtk_set_id_space(self._h, 1 if gpt2 else 0))

    def set_stage_timing(self, per_stage: bool) -> None:
        """Time every stage of a batch that runs in one piece (chunker, merge, scans, pack in ``stage_ms()``) instead
        of the pipeline as a whole; off by default because the extra events cost small calls about a tenth."""
        self._check(self._lib.gtk_set_stage_timing(self._h, 1 if per_stage else 0))

    def set_base_block_size(self, threads: int) -> None:
        """Threads per CTA of the one-CTA-per-chunk kernel (GTK_MODE_BASE): 0 = one warp per KiB of chunk,
        else 64, 128, 256, 512 or 1024 (the reference's BLOCK_SIZE).  Results never depend on it."""
        self._check(self._lib.gtk_set_base_block_size(self._h, int(threads)))

    def write_token_strings(self, path: str, ids, chunk_id_offsets) -> None:
        """One chunk per line, tokens as GPT-2 symbol strings separated by spaces (the reference's
        data/output/gpu_tokens_blockbpe.txt format)."""
        a = np.ascontiguousarray(ids, dtype=np.int32)
        off = np.ascontiguousarray(chunk_id_offsets, dtype=np.int64)
        self._check(self._lib.gtk_write_token_strings(self._h, os.fsencode(path), a.ctypes.data, off.ctypes.data,
                                                      len(off) - 1))

    # ------------------------------------------------------------------ host buffers
    def _result(self, copy: bool = True):
        n_ids, n_chunks, n_texts = C.c_int64(), C.c_int64(), C.c_int64()
        self._lib.gtk_result_sizes(self._h, C.byref(n_ids), C.byref(n_chunks), C.byref(n_texts))
        p_ids, p_text, p_chunk = C.c_void_p(), C.c_void_p(), C.c_void_p()
        self._lib.gtk_result_view(self._h, C.byref(p_ids), C.byref(p_text), C.byref(p_chunk))

        def view(ptr, n, ctype, dtype):
            if n == 0 or not ptr.value:
                return np.zeros(n, dtype=dtype)
            a = np.frombuffer((ctype * n).from_address(ptr.value), dtype=dtype)
            return a.copy() if copy else a

        ids = view(p_ids, n_ids.value, C.c_int32, np.int32)
        text_off = view(p_text, n_texts.value + 1, C.c_int64, np.int64)
        chunk_off = view(p_chunk, n_chunks.value + 1, C.c_int64, np.int64)
        return ids, text_off, chunk_off

    def encode(self, data, text_offsets=None, mode: int = GTK_MODE_OPT, copy: bool = True):
        """Tokenise host bytes.  ``data`` is one buffer; ``text_offsets`` (int64[T+1]) cuts it into
        texts (default: one text).  Returns (ids, text_id_offsets, chunk_id_offsets, kernel_ms)."""
        buf = _as_u8(data)
        if text_offsets is None:
            text_offsets = np.array([0, len(buf)], dtype=np.int64)
        off = np.ascontiguousarray(text_offsets, dtype=np.int64)
        ms = C.c_float()
        self._check(self._lib.gtk_encode(self._h, int(mode), buf.ctypes.data, off.ctypes.data, len(off) - 1,
                                         C.byref(ms)))
        ids, toff, coff = self._result(copy)
        return ids, toff, coff, ms.value

    def encode_texts(self, texts, mode: int = GTK_MODE_OPT):
        """list[bytes|str] -> (ids, text_id_offsets, chunk_id_offsets, kernel_ms)."""
        blobs = [t.encode("utf-8") if isinstance(t, str) else bytes(t) for t in texts]
        off = np.zeros(len(blobs) + 1, dtype=np.int64)
        if blobs:
            off[1:] = np.cumsum([len(b) for b in blobs])
        return self.encode(b"".join(blobs), off, mode)

    def encode_cpu(self, data, text_offsets=None, rule: int = GTK_RULE_GREEDY):
        buf = _as_u8(data)
        if text_offsets is None:
            text_offsets = np.array([0, len(buf)], dtype=np.int64)
        off = np.ascontiguousarray(text_offsets, dtype=np.int64)
        self._check(self._lib.gtk_encode_cpu(self._h, int(rule), buf.ctypes.data, off.ctypes.data, len(off) - 1))
        return self._result(True)

    # ------------------------------------------------------------------ device buffers
    def encode_device(self, d_bytes: int, n_bytes: int, d_text_offsets: int, n_texts: int, d_out_ids: int,
                      out_capacity: int, d_out_chunk_offsets: int = 0, chunk_capacity: int = 0,
                      mode: int = GTK_MODE_OPT):
        """Raw device pointers (ints) in and out.  Returns (n_ids, n_chunks, kernel_ms)."""
        n_ids, n_chunks, ms = C.c_int64(), C.c_int64(), C.c_float()
        self._check(self._lib.gtk_encode_device(self._h, int(mode), d_bytes, int(n_bytes), d_text_offsets,
                                                int(n_texts), d_out_ids, int(out_capacity),
                                                d_out_chunk_offsets or None, int(chunk_capacity),
                                                C.byref(n_ids), C.byref(n_chunks), C.byref(ms)))
        return n_ids.value, n_chunks.value, ms.value

    def encode_chunks_noalloc(self, d_bytes: int, n_bytes: int, d_chunk_offsets: int, n_chunks: int,
                              max_chunk_bytes: int, d_out_ids: int, d_out_counts: int) -> None:
        """Allocation-free variant for callers that may not allocate while tokenising (raw device
        pointers).  Ids of chunk c land at ``d_out_ids[chunk_offsets[c]:]``, their number in
        ``d_out_counts[c]``.  At most ``NOALLOC_MAX_CHUNK_BYTES`` bytes per chunk."""
        self._check(self._lib.gtk_encode_chunks_noalloc(self._h, d_bytes, int(n_bytes), d_chunk_offsets,
                                                        int(n_chunks), int(max_chunk_bytes), d_out_ids,
                                                        d_out_counts))

    # ------------------------------------------------------------------ decode
    def decode(self, ids) -> bytes:
        a = np.ascontiguousarray(ids, dtype=np.int32)
        n = C.c_int64()
        self._check(self._lib.gtk_decode(self._h, a.ctypes.data, len(a), None, 0, C.byref(n)))
        out = np.empty(max(n.value, 1), dtype=np.uint8)
        self._check(self._lib.gtk_decode(self._h, a.ctypes.data, len(a), out.ctypes.data, n.value, C.byref(n)))
        return out[:n.value].tobytes()

    def token_symbols(self, tid: int) -> bytes:
        buf = C.create_string_buffer(1024)
        n = self._lib.gtk_token_symbols(self._h, int(tid), buf, 1024)
        if n < 0:
            raise KeyError(tid)
        return buf.raw[:n]
