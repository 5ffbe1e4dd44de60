"""Builds ``libsinge_kernel_sys.so`` (the C-ABI library of hand-written sm_100a kernels) in-tree.

``python -m singe_b200.build`` compiles every ``csrc/*.cu`` with nvcc for ``sm_100a`` only and links
the objects into ``singe_b200/libsinge_kernel_sys.so``.  nvcc cross-compiles, so this works on a
machine without a GPU.  Objects are rebuilt only when their source (or a header) is newer.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libsinge_kernel_sys.so")

NVCC = os.environ.get("SINGE_NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-ccbin", "/usr/bin/g++",
]


def _newest_header() -> float:
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    return max(os.path.getmtime(h) for h in headers)


def _compile(source: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.basename(source)[:-3] + ".o")
    stamp = max(os.path.getmtime(source), _newest_header())
    if os.path.exists(obj) and os.path.getmtime(obj) >= stamp:
        return obj
    command = [NVCC, *FLAGS, "-c", source, "-o", obj]
    if verbose:
        command.insert(1, "-Xptxas=-v")
    result = subprocess.run(command, capture_output=True, text=True)
    if verbose and result.stderr:
        sys.stderr.write(result.stderr)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source}:\n{result.stdout}\n{result.stderr}")
    return obj


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    if force:
        for stale in glob.glob(os.path.join(OBJ, "*.o")):
            os.remove(stale)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(lambda s: _compile(s, verbose), sources))
    newest = max(os.path.getmtime(o) for o in objects)
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        command = [NVCC, "-shared", "-o", LIB, *objects, "-ccbin", "/usr/bin/g++", "-lcudart"]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
