"""ctypes binding of the in-tree native library ``_C/libdistdl_b200.so``.

The library has a plain C ABI (raw device pointers, sizes, a CUDA stream
handle), so it carries no dependency on the PyTorch C++ headers and builds
in seconds.  :func:`lib` loads it once; when a CUDA device is present and
the library is missing the import fails loudly instead of falling back to
eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_C", "libdistdl_b200.so")
# DISTDL_DEBUG_LIB=1 loads the bounds-checking build instead (python -m distdl_b200._build --debug)
if os.environ.get("DISTDL_DEBUG_LIB", "0") == "1":
    LIB_PATH = os.path.join(_HERE, "_C", "libdistdl_b200_debug.so")

_lock = threading.Lock()
_lib = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
c_fp = ctypes.POINTER(ctypes.c_float)

# name -> argtypes (restype is always int unless listed in _RESTYPES)
_SIGNATURES = {
    "dd_version": [],
    "dd_sm_count": [],
    "dd_read_status": [ctypes.POINTER(c_int)],
    "dd_read_wait_ns": [ctypes.POINTER(ctypes.c_ulonglong)],
    "dd_gemm_bf16": [c_void_p, c_int, c_ll, c_ll, c_void_p, c_int, c_ll, c_ll, c_void_p, c_ll, c_ll, c_void_p,
                     c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
    "dd_norm_bwd_parts": [c_int],
    "dd_norm_fwd": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                    c_float, c_void_p],
    "dd_norm_bwd": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                    c_void_p, c_int, c_int, c_int, c_void_p],
    "dd_swiglu_fwd": [c_void_p, c_void_p, c_ll, c_int, c_void_p],
    "dd_swiglu_bwd": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p],
    "dd_gelu_fwd": [c_void_p, c_void_p, c_ll, c_void_p],
    "dd_gelu_bwd": [c_void_p, c_void_p, c_void_p, c_ll, c_void_p],
    "dd_rope": [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_float, c_void_p],
    "dd_embedding_fwd": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_void_p],
    "dd_embedding_bwd": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_void_p],
    "dd_xent": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_float, c_void_p],
    "dd_adamw": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_float, c_float, c_float, c_float,
                 c_float, c_int, c_void_p, c_float, c_int, c_void_p],
    "dd_sumsq_f32": [c_void_p, c_ll, c_void_p, c_void_p],
    "dd_add_bf16": [c_void_p, c_void_p, c_void_p, c_ll, c_void_p],
    "dd_cast_f32_bf16": [c_void_p, c_void_p, c_ll, c_float, c_void_p],
    "dd_cast_bf16_f32": [c_void_p, c_void_p, c_ll, c_float, c_int, c_void_p],
}


class NativeError(RuntimeError):
    """A native entry point returned a non-zero status."""


_STATUS_NAMES = {
    1001: "bad argument",
    1002: "misaligned pointer or stride (16-byte alignment required)",
    1003: "size beyond the supported maximum",
    1004: "CUDA driver call failed",
    1005: "bounded device-side wait timed out",
    1006: "address outside the tensor's storage (bounds-checking build)",
}

# Counts launches of this library's kernels (every entry point launches at
# least one kernel); bench.py reports it.
launch_count = 0


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    """Returns the loaded library, loading (never building) it on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"native library {LIB_PATH} is missing: run `python -m distdl_b200._build` "
                "(nvcc cross-compiles for sm_100a without a GPU)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError:
                continue
            fn.argtypes = argtypes
            fn.restype = c_int
        _lib = handle
    return _lib


def declare(name: str, argtypes, restype=c_int):
    """Registers the signature of an entry point defined outside the table above."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = restype


def check(status: int, what: str = "") -> None:
    if status != 0:
        msg = _STATUS_NAMES.get(status)
        if msg is None:
            msg = f"CUDA error {status}"
        raise NativeError(f"{what}: {msg} (status {status})")


_nvtx = None


def _nvtx_module():
    """``torch.cuda.nvtx`` when ``DISTDL_NVTX=1`` (every native launch then sits in an NVTX
    range named after its entry point), else ``False``."""
    global _nvtx
    if _nvtx is None:
        _nvtx = False
        if os.environ.get("DISTDL_NVTX", "0") == "1":
            try:
                import torch
                _nvtx = torch.cuda.nvtx
            except Exception:       # noqa: BLE001
                _nvtx = False
    return _nvtx


def call(name: str, *args) -> None:
    """Calls an entry point and raises :class:`NativeError` on failure."""
    global launch_count
    launch_count += 1
    nvtx = _nvtx_module()
    if nvtx:
        nvtx.range_push(name)
        try:
            check(getattr(lib(), name)(*args), name)
        finally:
            nvtx.range_pop()
        return
    check(getattr(lib(), name)(*args), name)


def read_status():
    """Reads and clears the device-side status record of the current device.

    Returns ``(code, where, expected, seen)``; code 0 means that no kernel
    gave up a bounded wait since the last call.  Synchronises the device.
    """
    out = (c_int * 4)()
    check(lib().dd_read_status(out), "dd_read_status")
    return tuple(out)


WAIT_KINDS = ("ag_gemm: peer shard staged", "ag_gemm: peers done reading", "ag_gemm: row block arrived",
              "gemm_rs: slot consumed", "rs fold: peer delivered", "collectives: team barrier", "-", "-")


def read_wait_ns():
    """Reads and clears the per-kind totals of nanoseconds that designated
    threads spent waiting for other GPUs (diagnostics; synchronises the device)."""
    out = (ctypes.c_ulonglong * 8)()
    check(lib().dd_read_wait_ns(out), "dd_read_wait_ns")
    return dict(zip(WAIT_KINDS, (int(v) for v in out)))
