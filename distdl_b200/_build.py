"""Builds the native sm_100a library of distdl_b200 in-tree.

Every ``.cu`` / ``.cpp`` file under ``distdl_b200/csrc`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a`` (cross-compiles without a
GPU) and linked into ``distdl_b200/_C/libdistdl_b200.so``, a plain C-ABI
shared library that :mod:`distdl_b200._native` loads through ``ctypes``.
Run ``python -m distdl_b200._build`` (``--force`` to rebuild everything,
``-v`` to print the ptxas resource usage).
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
OUT_DIR = os.path.join(_HERE, "_C")
OBJ_DIR = os.path.join(CSRC, "build")
LIB_PATH = os.path.join(OUT_DIR, "libdistdl_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-fopenmp",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; cannot build the distdl_b200 native library")
    return cand


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))


def _headers_digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cuh", ".h", ".hpp")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile_one(src: str, verbose: bool, hdr: str, force: bool, debug: bool = False) -> str:
    obj = os.path.join(OBJ_DIR + ("_debug" if debug else ""), src.rsplit(".", 1)[0] + ".o")
    stamp = obj + ".stamp"
    with open(os.path.join(CSRC, src), "rb") as fh:
        digest = hashlib.sha256(fh.read() + hdr.encode()).hexdigest()
    if not force and os.path.exists(obj) and os.path.exists(stamp):
        with open(stamp) as fh:
            if fh.read().strip() == digest:
                return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *(["-DDD_BOUNDS_CHECK"] if debug else []), "-I", CSRC, "-c", os.path.join(CSRC, src),
           "-o", obj]
    if src.endswith(".cpp"):
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    with open(stamp, "w") as fh:
        fh.write(digest)
    return obj


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> str:
    """Compiles what changed and links the shared library; returns its path.  ``debug`` builds the
    bounds-checking variant (``-DDD_BOUNDS_CHECK``: kernels that address tensors through computed
    offsets check every address against the tensor's storage, record a violation in the status
    record and skip the access) as ``libdistdl_b200_debug.so``; ``DISTDL_DEBUG_LIB=1`` loads it."""
    os.makedirs(OBJ_DIR + ("_debug" if debug else ""), exist_ok=True)
    os.makedirs(OUT_DIR, exist_ok=True)
    hdr = _headers_digest()
    srcs = _sources()
    lib_path = LIB_PATH.replace(".so", "_debug.so") if debug else LIB_PATH
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose, hdr, force, debug), srcs))
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(lib_path) or os.path.getmtime(lib_path) < newest:
        cmd = [_nvcc(), "-shared", "-o", lib_path, *objs, "-Xcompiler", "-fopenmp", "-lgomp",
               "-gencode", "arch=compute_100a,code=sm_100a"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug="--debug" in sys.argv)
    print(path)
