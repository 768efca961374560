"""Ahead-of-time build of the CUDA library for sm_100a (replaces the reference's runtime nvcc JIT,
``green_attention/jit.py:139-183``): one ``nvcc`` call over ``csrc/api.cu`` producing
``greenattention_b200/_lib/libgreen_attention.so`` in the source tree. nvcc cross-compiles, so no GPU is needed.

    python -m greenattention_b200.build [--force] [--verbose]
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
LIB_DIR = os.path.join(PKG, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libgreen_attention.so")
STAMP = os.path.join(LIB_DIR, "build.stamp")

FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", 
    "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: set CUDA_HOME")
    return found


def _sources():
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".h"))]
    files.append(os.path.join(INCLUDE, "green_attention.h"))
    return files


def _identity() -> str:
    h = hashlib.sha256(" ".join(FLAGS).encode())
    for f in _sources():
        with open(f, "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    ident = _identity()
    if not force and os.path.exists(LIB_PATH) and os.path.exists(STAMP) and open(STAMP).read().strip() == ident:
        return LIB_PATH
    cmd = [_nvcc(), *FLAGS, "-I", INCLUDE, "-o", LIB_PATH, os.path.join(CSRC, "api.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode:
        raise RuntimeError("nvcc failed building libgreen_attention.so")
    with open(STAMP, "w") as f:
        f.write(ident)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
