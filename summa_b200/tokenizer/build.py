"""Builds the native tokenizer core in-tree: `python -m summa_b200.tokenizer.build` compiles
`csrc/fast_bpe.cpp` with g++ into `libsumma_tokenizer.so` next to this file (host code only, no CUDA)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc", "fast_bpe.cpp")
LIB = os.path.join(HERE, "libsumma_tokenizer.so")


def build(force: bool = False) -> str:
    deps = [SRC, os.path.join(HERE, "csrc", "unicode_tables.h")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) > os.path.getmtime(d) for d in deps):
        return LIB
    cmd = [os.environ.get("CXX", "g++"), "-O3", "-std=c++17", "-fPIC", "-shared", "-pthread", "-Wall", "-o", LIB, SRC]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("g++ failed for the tokenizer core")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
