"""Small helpers shared by the op wrappers."""
from __future__ import annotations

import os

import torch

from .. import _native


def stream_ptr(t: torch.Tensor = None) -> int:
    """Raw handle of the current CUDA stream (kernels launch on torch's stream)."""
    return torch.cuda.current_stream().cuda_stream


def ptr(t):
    return 0 if t is None else t.data_ptr()


def use_native(*tensors) -> bool:
    """True when the operands live on a CUDA device: the hand-written kernels run.

    CPU tensors take the plain PyTorch path, which exists for the gloo
    plumbing and adjoint tests only.  On a CUDA device a missing native
    library is an error, never a silent fallback.
    """
    if os.environ.get("DISTDL_FORCE_TORCH", "0") == "1":
        return False            # baseline arm: library kernels (cuBLAS / cuDNN / ATen) everywhere
    for t in tensors:
        if t is not None and t.is_cuda:
            if not _native.available():
                raise ImportError("distdl_b200 native library missing on a CUDA machine; "
                                  "run `python -m distdl_b200._build`")
            return True
    return False
