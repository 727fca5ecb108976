"""Array-level Python access to the C ABI of the B200 tokenizer (ctypes).

The drop-in class with the reference's method names lives in the compiled
module ``gputok_gpu`` (pybind11, next to this package); this package is the
array-level companion used by the benchmark, the multi-GPU driver and the
tests: host-buffer and device-buffer encodes, the synthetic text generator
and the shard planner.

There is no CPU fallback: importing works everywhere, but every GPU entry
point raises if the CUDA library is missing or no device is present.
"""
from .capi import (GTK_MODE_BASE, GTK_MODE_LOCALMIN, GTK_MODE_OPT, GTK_RULE_GREEDY, GTK_RULE_LOCALMIN, GtkError, Tokenizer,
                   library_path, load_library)
from .shards import partition_by_bytes, stitch_offsets
from .textgen import MIX_PLAIN, MIX_STRESS, TextGen

__all__ = [
    "GTK_MODE_BASE", "GTK_MODE_LOCALMIN", "GTK_MODE_OPT", "GTK_RULE_GREEDY", "GTK_RULE_LOCALMIN", "GtkError", "Tokenizer",
    "library_path", "load_library", "partition_by_bytes", "stitch_offsets", "MIX_PLAIN", "MIX_STRESS", "TextGen",
]
