"""Builds libllm_cuda.so (the C-ABI library of include/llm_cuda.h) in-tree with nvcc for sm_100a.

`python -m scriptonait_b200._build [--force] [--verbose]`. nvcc cross-compiles without a GPU.
-fmad=false: the sampler's arithmetic must round exactly where the reference's f32
code rounds (no fused multiply-add, no fast-math).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIBRARY = os.path.join(LIBDIR, "libllm_cuda.so")
# the same sources with -DLLM_CUDA_CHECKED: stores at computed shared-memory / scratch offsets are compared with their
# bounds first (a violation sets a status bit and skips the store). The tests run small and odd shapes against it.
CHECKED_LIBRARY = os.path.join(LIBDIR, "libllm_cuda_checked.so")
SOURCES = ["sampler_kernels.cu", "stream_variants_f32.cu", "stream_variants_f32_tables.cu", "stream_variants_bf16.cu",
           "stream_variants_bf16_tables.cu", "llm_cuda_api.cu", "no_alloc.cu", "lm_head.cu", "cross_entropy.cu"]
HEADERS = ["sampler_kernels.h", "sampler_device.cuh", "lm_head.h", "cross_entropy.h", os.path.join("..", "..", "include", "llm_cuda.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true", "-ftz=false",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared",
    "--threads", "0",   # the translation units compile side by side (the streaming kernel's variants are four of them)
]


def _sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def is_stale(library: str = LIBRARY) -> bool:
    if not os.path.exists(library):
        return True
    built = os.path.getmtime(library)
    deps = _sources() + [os.path.normpath(os.path.join(CSRC, h)) for h in HEADERS]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def nvcc_path() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libllm_cuda.so cannot be built")


def _command(library: str, checked: bool, verbose: bool) -> list[str]:
    cmd = [nvcc_path(), *NVCC_FLAGS]
    if checked:
        cmd += ["-DLLM_CUDA_CHECKED"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    return cmd + _sources() + ["-o", library]


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    library = CHECKED_LIBRARY if checked else LIBRARY
    if not (force or is_stale(library)):
        return library
    os.makedirs(LIBDIR, exist_ok=True)
    subprocess.run(_command(library, checked, verbose), check=True)
    return library


def build_all(force: bool = False) -> list[str]:
    """The product library and the checked one, compiled side by side."""
    os.makedirs(LIBDIR, exist_ok=True)
    jobs = [(lib, subprocess.Popen(_command(lib, chk, False)))
            for lib, chk in ((LIBRARY, False), (CHECKED_LIBRARY, True)) if force or is_stale(lib)]
    for lib, proc in jobs:
        if proc.wait() != 0:
            raise RuntimeError(f"nvcc failed for {lib}")
    return [LIBRARY, CHECKED_LIBRARY]


if __name__ == "__main__":
    if "--all" in sys.argv:
        print("\n".join(build_all(force="--force" in sys.argv)))
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, checked="--checked" in sys.argv))
