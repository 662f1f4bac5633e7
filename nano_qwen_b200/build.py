"""Builds ``libnq_fp8.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m nano_qwen_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libnq_fp8.so")
SOURCES = ["nq_quant.cu", "nq_gemm.cu", "nq_capi.cu", "nq_noalloc.cu", "nq_p2p.cu", "nq_sym.cu", "nq_fused_quant.cu"]
HEADERS = ["nq_ptx.cuh", "nq_internal.cuh", os.path.join("..", "..", "include", "nq_fp8.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def source_hash() -> str:
    """sha256 over the CUDA sources and headers the library is built from (names and contents, fixed order)."""
    h = hashlib.sha256()
    for f in SOURCES + HEADERS:
        h.update(os.path.basename(f).encode() + b"\0")
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:32]


def built_hash() -> str | None:
    """The source hash compiled into the existing library (``nq_source_hash``), or None if there is no usable library."""
    if not os.path.exists(LIB_PATH):
        return None
    import ctypes
    try:
        lib = ctypes.CDLL(LIB_PATH)
        fn = lib.nq_source_hash
    except (OSError, AttributeError):
        return None
    fn.restype = ctypes.c_char_p
    return fn().decode()


def _stale() -> bool:
    return built_hash() != source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library unless the one in the tree was built from exactly the present sources; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libnq_fp8.so")
    cmd = [nvcc, *NVCC_FLAGS, f'-DNQ_SOURCE_HASH="{source_hash()}"', "-o", LIB_PATH, *SOURCES]
    proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
