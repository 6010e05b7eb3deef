"""Sliding-window (local) causal attention over a sequence split across workers, by halo exchange.

New relative to the reference, which notes that ``HaloExchange`` could express the neighbour
traffic of windowed attention but has no attention code.  With a window of ``w`` tokens a query
attends to itself and the ``w - 1`` tokens before it, so a worker only ever needs the last
``w - 1`` keys / values of its LEFT neighbour: K and V get a ghost region of that width on the left
of the sequence dimension, one :class:`~distdl_b200.nn.HaloExchange` each fills it (its adjoint
returns the gradients of the ghost keys to their owner), and a banded causal mask does the rest.
Communication per layer is ``2 (w - 1) * heads * head_dim`` elements per worker whatever the
sequence length, against the whole K / V for ring or all-to-all attention.
"""
import math

import numpy as np
import torch

from .halo_exchange import HaloExchange
from .module import Module


class DistributedSlidingWindowAttention(Module):
    r"""``forward(q, k, v) -> out`` with ``q [b, s_local, Hq, D]``, ``k, v [b, s_local, Hkv, D]`` on
    ``P_seq = [B, S, H, 1]`` (contiguous sequence blocks in worker order).  Query ``i`` attends to the
    keys ``i - window + 1 .. i`` of the GLOBAL sequence.  ``window - 1`` must not exceed the
    neighbour's block length.  The local product is the library attention with an explicit mask."""

    def __init__(self, P_seq, window, scale=None, buffer_manager=None):
        super().__init__()
        self.P_seq = P_seq
        self.window, self.scale = int(window), scale
        if self.window < 1:
            raise ValueError("window must be at least 1")
        if not P_seq.active:
            return
        if P_seq.dim != 4 or int(P_seq.shape[3]) != 1:
            raise ValueError("DistributedSlidingWindowAttention expects a partition of shape [B, S, H, 1]")
        self.has_left = int(P_seq.index[1]) > 0
        w = self.window - 1 if self.has_left else 0
        self.ghost = w
        halo = np.zeros((4, 2), dtype=int)
        halo[1, 0] = w                                   # ghost keys on the left of the sequence dimension
        recv = halo.copy()
        send = np.zeros((4, 2), dtype=int)
        if int(P_seq.index[1]) < int(P_seq.shape[1]) - 1:
            send[1, 1] = self.window - 1                 # my last keys go to the right-hand neighbour
        bm = buffer_manager or self._distdl_backend.BufferManager()
        self.halo_k = HaloExchange(P_seq, halo, recv, send, bm)
        self.halo_v = HaloExchange(P_seq, halo, recv, send, bm)

    def forward(self, q, k, v):
        if not self.P_seq.active:
            return q
        b, s, hq, d = q.shape
        hkv = k.shape[2]
        g, w = self.ghost, self.window
        if int(self.P_seq.shape[1]) > 1 and w - 1 > s:
            raise ValueError(f"window - 1 = {w - 1} exceeds the block length {s}")
        if int(self.P_seq.shape[1]) > 1:
            pad = (0, 0, 0, 0, g, 0)                     # left of the sequence dimension
            k = self.halo_k(torch.nn.functional.pad(k, pad))
            v = self.halo_v(torch.nn.functional.pad(v, pad))
        # key j of the padded block sits at local position j - g; query i sees i - w < j - g <= i
        qi = torch.arange(s, device=q.device).unsqueeze(1)
        kj = torch.arange(s + g, device=q.device).unsqueeze(0) - g
        mask = (kj <= qi) & (kj > qi - w)
        rep = hq // hkv
        kh = k.transpose(1, 2).repeat_interleave(rep, dim=1) if rep > 1 else k.transpose(1, 2)
        vh = v.transpose(1, 2).repeat_interleave(rep, dim=1) if rep > 1 else v.transpose(1, 2)
        scale = self.scale if self.scale is not None else 1.0 / math.sqrt(d)
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), kh, vh, attn_mask=mask, scale=scale)
        return o.transpose(1, 2)
