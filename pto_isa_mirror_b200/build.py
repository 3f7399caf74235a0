"""In-tree build of libpto_b200.so (nvcc, sm_100a only).

Run as ``python -m pto_isa_mirror_b200.build``. The library lands in ``pto_isa_mirror_b200/lib/`` next to the
sources so that it travels with the source tree; nothing is written outside the package directory.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB = os.path.join(LIB_DIR, "libpto_b200.so")
SOURCES = ["pto_b200_capi.cu"]
HEADERS = ["gemm_tile_loop.cuh", "gemm_tile_loop_2cta.cuh", "gemv.cuh", "gemv_mx.cuh", "ksplit_reduce.cuh", "mx_quantize.cuh",
           "sm100_ptx.cuh", os.path.join("..", "..", "include", "pto_b200.h")]

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    deps = [os.path.join(CSRC, s) for s in SOURCES] + [os.path.normpath(os.path.join(CSRC, h)) for h in HEADERS]
    return _newest(deps) > os.path.getmtime(LIB)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources into lib/libpto_b200.so and return its path."""
    if not force and not needs_build():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
