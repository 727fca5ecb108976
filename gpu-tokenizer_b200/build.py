"""Build the native parts in-tree (no JIT cache, the .so files sit beside the sources).

    python build.py            # everything
    python build.py --force    # rebuild even if up to date

  libgputok_b200.so   CUDA kernels + C ABI (nvcc, sm_100a only)
  libgputok_b200_checked.so   the same built with -DGTK_CHECKED: every data-dependent index into shared
                      memory and the work buffers is range-checked, violations are recorded and skipped
  libgtk_textgen.so   seeded synthetic text generator (gcc, CPU only)
  gputok_gpu*.so      pybind11 module exposing the reference's GpuTokenizer surface (g++)
  gpu_tokenizer_blockbpe  command-line front end with the reference binary's arguments and output (g++)
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

LIB = os.path.join(HERE, "libgputok_b200.so")
LIB_CHECKED = os.path.join(HERE, "libgputok_b200_checked.so")
TEXTGEN = os.path.join(HERE, "libgtk_textgen.so")
PYMOD = os.path.join(HERE, "gputok_gpu" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
CLI = os.path.join(HERE, "gpu_tokenizer_blockbpe")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared"]


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str]) -> None:
    print("+", " ".join(cmd), flush=True)
    subprocess.run(cmd, check=True, cwd=HERE)


def build_cuda(force: bool = False, ptxas_verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, f) for f in ("gtk_kernels.cu", "gtk_api.cu", "gtk_table.cpp")]
    deps = srcs + [os.path.join(CSRC, f) for f in ("gtk_device.cuh", "gtk_table.hpp")] + \
        [os.path.join(INCLUDE, "gputok_b200.h")]
    if force or _stale(LIB, deps):
        nvcc = os.environ.get("NVCC", "nvcc")
        extra = ["-Xptxas", "-v"] if ptxas_verbose else []
        _run([nvcc] + NVCC_FLAGS + extra + srcs + ["-o", LIB])
    return LIB


def build_cuda_checked(force: bool = False) -> str:
    """The bounds-checked build (stands in for a memory sanitizer, which this pool does not offer)."""
    srcs = [os.path.join(CSRC, f) for f in ("gtk_kernels.cu", "gtk_api.cu", "gtk_table.cpp")]
    deps = srcs + [os.path.join(CSRC, f) for f in ("gtk_device.cuh", "gtk_table.hpp")] + \
        [os.path.join(INCLUDE, "gputok_b200.h")]
    if force or _stale(LIB_CHECKED, deps):
        nvcc = os.environ.get("NVCC", "nvcc")
        _run([nvcc] + NVCC_FLAGS + ["-DGTK_CHECKED"] + srcs + ["-o", LIB_CHECKED])
    return LIB_CHECKED


def build_textgen(force: bool = False) -> str:
    src = os.path.join(CSRC, "gtk_textgen.c")
    if force or _stale(TEXTGEN, [src]):
        _run(["gcc", "-O3", "-std=gnu11", "-fPIC", "-shared", "-fvisibility=hidden", src, "-o", TEXTGEN,
              "-lm", "-lpthread"])
    return TEXTGEN


def build_pymod(force: bool = False) -> str:
    import pybind11

    src = os.path.join(CSRC, "gputok_pybind.cpp")
    if force or _stale(PYMOD, [src, os.path.join(INCLUDE, "gputok_b200.h"), LIB]):
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
              "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], src,
              "-L", HERE, "-lgputok_b200", "-Wl,-rpath,$ORIGIN", "-o", PYMOD])
    return PYMOD


def build_cli(force: bool = False) -> str:
    """Command-line front end with the reference binary's arguments and output lines."""
    src = os.path.join(CSRC, "gpu_tokenizer_blockbpe.cpp")
    if force or _stale(CLI, [src, os.path.join(INCLUDE, "gputok_b200.h"), LIB]):
        _run(["g++", "-O2", "-std=c++17", src, "-L", HERE, "-lgputok_b200", "-Wl,-rpath,$ORIGIN", "-o", CLI])
    return CLI


def build_all(force: bool = False) -> None:
    build_cuda(force)
    build_cuda_checked(force)
    build_textgen(force)
    build_pymod(force)
    build_cli(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
