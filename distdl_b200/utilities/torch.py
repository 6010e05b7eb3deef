"""Tensor helpers: zero-volume tensors (the "this worker holds nothing"
sentinel), tensor structure records, padding format conversion.
Reference: ``src/distdl/utilities/torch.py:5-49``."""
from __future__ import annotations

import numpy as np
import torch


def zero_volume_tensor(b=None, dtype=None, requires_grad=False, device=None):
    """Empty tensor of shape ``(0,)``, or ``(b, 0)`` when a batch size is kept."""
    if dtype is None:
        dtype = torch.get_default_dtype()
    shape = (0,) if b is None else (int(b), 0)
    return torch.empty(shape, dtype=dtype, requires_grad=requires_grad, device=device)


class TensorStructure:
    """(shape, dtype, requires_grad) of a tensor; comparable, cheap to ship."""

    def __init__(self, tensor=None):
        self.shape = None
        self.dtype = None
        self.requires_grad = None
        if tensor is not None:
            self.fill_from_tensor(tensor)

    def fill_from_tensor(self, tensor):
        self.shape = tensor.shape
        self.dtype = tensor.dtype
        self.requires_grad = tensor.requires_grad

    def __eq__(self, other):
        if not isinstance(other, TensorStructure):
            return NotImplemented
        a = None if self.shape is None else tuple(int(s) for s in self.shape)
        b = None if other.shape is None else tuple(int(s) for s in other.shape)
        return a == b and self.dtype == other.dtype and self.requires_grad == other.requires_grad

    def __repr__(self):
        return f"TensorStructure(shape={self.shape}, dtype={self.dtype}, requires_grad={self.requires_grad})"


def distdl_padding_to_torch_padding(pad):
    """``[[a_0, b_0], ..., [a_n, b_n]]`` -> ``(a_n, b_n, ..., a_0, b_0)`` as ``F.pad`` wants."""
    pairs = np.asarray(pad, dtype=int).reshape(-1, 2)
    return tuple(int(v) for v in pairs[::-1].reshape(-1))
