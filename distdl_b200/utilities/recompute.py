"""Saved tensors that are rebuilt in the backward pass instead of being stored.

``with saved_as_recipe(t, fn): y = layer(t)`` makes every autograd function that runs
inside the block and saves ``t`` (or a view of its storage) for its backward keep a
*recipe* instead: ``fn`` is called when the backward pass asks for the tensor, and the
result stands in for ``t``.  Once the caller drops its own reference, ``t`` is freed
right after the forward pass.  Two uses in this package:

* outputs of cheap operators (norms, SwiGLU / GELU) that the following GEMM saves as its
  input: recomputing them costs one memory-bound kernel, storing them costs as much
  memory as the activation itself;
* the gathered weight of a ZeRO-3 layer: the backward pass gathers the shards again
  instead of holding the unsharded weight from forward to backward (what the
  reference's ``checkpoint=True`` does for its linear layers,
  ``src/distdl/nn/linear_ag_zero.py:21-77``).

Recipes are active only inside ``enabled()``; elsewhere ``saved_as_recipe`` does
nothing, so layers may call it unconditionally.  PyTorch applies only the innermost pair of
saved-tensor hooks, therefore all open recipes share one registry that every pair of
hooks consults.
"""
from __future__ import annotations

import contextlib
import weakref

import torch

_enabled = 0
_norms, _activation = True, True    # which cheap operator outputs recipes stand in for (besides gathered weights)
_targets = []          # open recipes, innermost last


def active() -> bool:
    return _enabled > 0


def rebuilds_norm_outputs() -> bool:
    """Inside ``enabled()``: whether norm outputs are rebuilt in the backward pass."""
    return _enabled > 0 and _norms


def rebuilds_activation_output() -> bool:
    """Inside ``enabled()``: whether the activation function's output is rebuilt in the backward pass."""
    return _enabled > 0 and _activation


def rebuilds_outputs() -> bool:
    return rebuilds_norm_outputs() or rebuilds_activation_output()


@contextlib.contextmanager
def enabled(flag: bool = True, norms: bool = True, activation: bool = True):
    """Turns recipes on (or, with ``flag=False``, off) for the duration of the block.  A caller with
    memory to spare keeps the re-gathering of ZeRO weights but stores the outputs of cheap operators
    after all: ``norms=False`` / ``activation=False``."""
    global _enabled, _norms, _activation
    before = (_enabled, _norms, _activation)
    _enabled = (before[0] + 1) if flag else 0
    _norms, _activation = norms, activation
    try:
        yield
    finally:
        _enabled, _norms, _activation = before


class Recipe:
    """``fn()`` rebuilds the tensor (called without gradient tracking).  The result is cached
    weakly, so that two saved views of one tensor asked for in the same backward step share one
    rebuild."""

    def __init__(self, fn):
        self.fn = fn
        self._ref = None
        self.rebuilds = 0

    def get(self):
        t = self._ref() if self._ref is not None else None
        if t is None:
            with torch.no_grad(), enabled(False):
                t = self.fn()
            self.rebuilds += 1
            self._ref = weakref.ref(t)
        return t


class _Packed:
    __slots__ = ("recipe", "shape", "stride", "offset")

    def __init__(self, recipe, shape, stride, offset):
        self.recipe, self.shape, self.stride, self.offset = recipe, shape, stride, offset


def _pack(t):
    if isinstance(t, torch.Tensor) and t.numel():
        ptr = t.untyped_storage().data_ptr()
        for ptr0, dtype, device, off0, recipe in reversed(_targets):
            if ptr == ptr0 and t.dtype == dtype and t.device == device:
                return _Packed(recipe, tuple(t.shape), tuple(t.stride()), t.storage_offset() - off0)
    return t


def _unpack(obj):
    if isinstance(obj, _Packed):
        base = obj.recipe.get()
        return torch.as_strided(base, obj.shape, obj.stride, base.storage_offset() + obj.offset)
    return obj


@contextlib.contextmanager
def saved_as_recipe(tensor, fn):
    """Inside the block, autograd saves ``fn`` wherever it would save ``tensor`` (any view of its
    storage).  ``fn`` must return a tensor with the layout of ``tensor``.  Does nothing when recipes
    are off, when ``fn`` is None or when ``tensor`` is empty."""
    if not active() or fn is None or not isinstance(tensor, torch.Tensor) or tensor.numel() == 0:
        yield None
        return
    recipe = Recipe(fn)
    _targets.append((tensor.untyped_storage().data_ptr(), tensor.dtype, tensor.device, tensor.storage_offset(), recipe))
    try:
        with torch.autograd.graph.saved_tensors_hooks(_pack, _unpack):
            yield recipe
    finally:
        _targets.pop()
