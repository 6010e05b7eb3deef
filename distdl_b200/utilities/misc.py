"""Odds and ends: stream barrier, attribute dict, dummy autograd context."""
from __future__ import annotations

import torch


def stream_barrier(stream):
    """Makes the current CUDA stream wait for everything queued on ``stream``."""
    if stream is not None and torch.cuda.is_available():
        torch.cuda.current_stream().wait_stream(stream)


class Bunch(dict):
    """dict whose items are also attributes."""

    def __getattr__(self, key):
        try:
            return self[key]
        except KeyError as e:
            raise AttributeError(key) from e

    def __setattr__(self, key, value):
        self[key] = value


class DummyContext(Bunch):
    """Stand-in for an autograd ``ctx`` so Function.forward/backward bodies can
    be exercised outside of autograd."""

    def save_for_backward(self, *tensors):
        self["saved_tensors"] = tensors

    def mark_dirty(self, *tensors):
        self["dirty_tensors"] = tensors

    def mark_non_differentiable(self, *tensors):
        self["non_differentiable"] = tensors

    def set_materialize_grads(self, value):
        self["materialize_grads"] = value
