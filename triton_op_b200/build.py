"""In-tree build of the CUDA library (``python -m triton_op_b200.build``).

One nvcc invocation turns ``csrc/pa_decode_sm100.cu`` into ``lib/libpa_decode_sm100.so`` for
sm_100a.  nvcc cross-compiles, so this also runs on a machine without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libpa_decode_sm100.so")
SOURCES = ["pa_decode_sm100.cu"]
HEADERS = ["pa_common.cuh", "pa_params.cuh", "pa_partition_fp8.cuh", "pa_partition_bf16.cuh", "pa_partition_tc.cuh", "pa_tcgen05.cuh",
           "pa_reduce.cuh", "pa_cache_write.cuh", "pa_exchange.cuh", "pa_stream_probe.cuh",
           os.path.join("..", "..", "include", "pa_decode_sm100.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: cannot build the sm_100a library")
    return exe


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [os.path.join(CSRC, h) for h in HEADERS]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; returns its path.
    ``trace`` adds the instantiations that stamp SM clocks into ``PaDecodeParams.trace`` (tuning aid)."""
    if not force and not needs_build():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + (["-DPA_TRACE_BUILD"] if trace else [])
    cmd += ["-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv or "--trace" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))
