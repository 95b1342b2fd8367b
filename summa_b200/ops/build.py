"""Builds the native kernel library in-tree with nvcc for sm_100a.

`python -m summa_b200.ops.build` compiles every `csrc/*.cu` to an object under
`_build/` (skipping objects newer than their sources and headers) and links
`libsumma_b200.so` next to this file. The kernels use only the CUDA runtime, so
the library loads through ctypes without pulling in the PyTorch headers, and
cross-compiles on a machine without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libsumma_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newest_header_mtime() -> float:
    return max((os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC)
                if f.endswith((".cuh", ".h"))), default=0.0)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(BUILD, os.path.splitext(os.path.basename(src))[0] + ".o")
    stamp = max(os.path.getmtime(src), _newest_header_mtime(), os.path.getmtime(__file__))
    if os.path.exists(obj) and os.path.getmtime(obj) > stamp:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"nvcc failed for {src}")
    if verbose:
        log = os.path.join(BUILD, os.path.basename(src) + ".ptxas.txt")
        with open(log, "w") as f:
            f.write(r.stdout + r.stderr)
    return obj


def build(verbose: bool = True, force: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    sources = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    if force:
        for f in os.listdir(BUILD):
            if f.endswith(".o"):
                os.remove(os.path.join(BUILD, f))
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), sources))
    if (not os.path.exists(LIB)) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
