"""Builds libsamq.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Run as ``python -m sam_quantization_b200.build``.  nvcc cross-compiles, so no GPU is
needed to build.  Each source is compiled to its own object (in parallel, and only when it or a
header changed); the objects are then linked into the shared library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libsamq.so")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def sources() -> list:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libsamq.so cannot be built")
    return exe


def _headers_mtime() -> float:
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(PKG_DIR, "..", "include", "samq.h"))
    return max(os.path.getmtime(d) for d in deps)


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n" + res.stdout + res.stderr)
    return res.stderr


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/*.cu into sam_quantization_b200/libsamq.so and return its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr = _headers_mtime()
    todo = []
    for src in sources():
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        newest = max(hdr, os.path.getmtime(os.path.join(CSRC, src)))
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < newest:
            todo.append(src)
    if todo:
        with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 1)) as pool:
            for src, log in zip(todo, pool.map(lambda s: _compile(s, verbose), todo)):
                if verbose:
                    sys.stderr.write(f"==== {src}\n{log}")
    objs = [os.path.join(OBJ_DIR, s[:-3] + ".o") for s in sources()]
    if todo or not os.path.exists(LIB_PATH) or any(os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs):
        res = subprocess.run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", LIB_PATH],
                             capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
