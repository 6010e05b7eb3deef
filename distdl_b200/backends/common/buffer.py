"""Growable staging buffers shared between layers
(``src/distdl/backends/common/buffer.py:7-149``).

An :class:`ExpandableBuffer` owns one flat tensor and hands out shaped views
of its head; asking for a view larger than the capacity reallocates (contents
kept, existing views re-pointed).  A :class:`BufferManager` keeps a list of
buffers per dtype (and per device) so that many layers reuse the same staging
memory; the allocation function is pluggable.  HaloExchange and Repartition pack
into and receive into these views on the transports that move whole messages
(gloo, NCCL).  The native transport needs none of them: its exchange kernel packs
straight into the receiving GPU's inbox, a region of the peer-mapped symmetric heap
that every process allocates once (``parallel/symm.py``); growing a peer-mapped
buffer on demand would be a collective over all processes in the middle of a layer's
lazy set-up, which inactive workers never enter.
"""
from __future__ import annotations

import numpy as np
import torch


class ExpandableBuffer:
    def __init__(self, dtype, initial_capacity=0, device=None, allocator=None):
        self.dtype = dtype
        self.device = device if device is not None else torch.device("cpu")
        self._allocator = allocator or (lambda n, dt, dev: torch.empty(n, dtype=dt, device=dev))
        self.capacity = int(initial_capacity)
        self.raw_buffer = self._allocator(self.capacity, self.dtype, self.device)
        self.views = {}

    def expand(self, new_capacity):
        new_capacity = int(new_capacity)
        if new_capacity <= self.capacity:
            return
        fresh = self._allocator(new_capacity, self.dtype, self.device)
        if self.capacity:
            fresh[: self.capacity].copy_(self.raw_buffer)
        self.raw_buffer = fresh
        self.capacity = new_capacity
        for shape in list(self.views):
            self.views[shape] = self._view(shape)

    def _view(self, shape):
        n = int(np.prod(shape)) if len(shape) else 1
        return self.raw_buffer[:n].view(shape)

    def allocate_view(self, view_shape):
        shape = tuple(int(s) for s in view_shape)
        n = int(np.prod(shape)) if len(shape) else 1
        if n > self.capacity:
            self.expand(n)
        self.views[shape] = self._view(shape)

    def get_view(self, view_shape):
        shape = tuple(int(s) for s in view_shape)
        if shape not in self.views:
            self.allocate_view(shape)
        return self.views[shape]


class BufferManager:
    def __init__(self, device=None, allocator=None):
        self.device = device
        self._allocator = allocator
        self.buffers_map = {}

    def request_buffers(self, n_buffers, dtype, **kwargs):
        device = kwargs.get("device", None)
        device = self.device if device is None else device
        on_host = device is None or torch.device(device).type == "cpu"
        # one pool per dtype, as in the reference; device tensors get pools of their own
        pool = self.buffers_map.setdefault(dtype if on_host else (dtype, str(torch.device(device))), [])
        while len(pool) < n_buffers:
            pool.append(ExpandableBuffer(dtype, 0, device=device, allocator=self._allocator))
        return pool[:n_buffers]


# names used by the reference
MPIExpandableBuffer = ExpandableBuffer
MPIBufferManager = BufferManager
