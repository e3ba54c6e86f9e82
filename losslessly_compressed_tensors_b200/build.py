"""Compile the CUDA sources into ``liblct_b200.so`` next to this file (sm_100a only).

    python -m losslessly_compressed_tensors_b200.build [--force] [--verbose]

The library is built in-tree so that it travels with the checkout; nothing is
JIT-compiled at import time.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIBRARY = os.path.join(HERE, "liblct_b200.so")
SOURCES = ("capi.cu", "tables.cu", "arena.cu", "encode.cu", "decode.cu", "update.cu")


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build liblct_b200.so")
    return found


def _stale() -> bool:
    if not os.path.exists(LIBRARY):
        return True
    built = os.path.getmtime(LIBRARY)
    inputs = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    inputs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return any(os.path.getmtime(path) > built for path in inputs)


def build(force: bool = False, verbose: bool = False) -> str:
    """Build the shared library if missing or older than its sources; return its path."""
    if not force and not _stale():
        return LIBRARY
    # Link into a private name and move it into place: another process (a second rank of the same
    # job, a test worker) never maps a half-written library, and a failed build leaves the old one.
    partial = f"{LIBRARY}.{os.getpid()}.partial"
    command = [
        _nvcc(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
        "-Xcompiler", "-fPIC", "-shared", "-I", INCLUDE, "-I", CSRC,
        "-o", partial, *[os.path.join(CSRC, name) for name in SOURCES],
    ]
    if verbose:
        command[1:1] = ["-Xptxas", "-v"]
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose or result.returncode:
        sys.stderr.write(result.stdout + result.stderr)
    if result.returncode:
        if os.path.exists(partial):
            os.remove(partial)
        raise RuntimeError("nvcc failed building liblct_b200.so")
    os.replace(partial, LIBRARY)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
