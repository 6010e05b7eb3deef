"""Expert-parallel dispatch / combine over peer memory.

``dispatch``: the rows of the routed (token, choice) pairs are written straight into the
capacity buffers of the GPUs that own the chosen experts (peer stores from inside one
kernel), in the ``[local expert, source GPU * capacity, d]`` layout that the grouped expert
GEMM reads.  ``combine``: every GPU reads the expert outputs of its own pairs straight from
the owners' buffers and forms the weighted sum per token.  Each replaces a permutation
kernel + an all-to-all + a transposing copy of the unfused path
(:mod:`distdl_b200.ops.moe` + ``all_to_all``).  The reference has no routing code at all
(``src/distdl/nn/linear_ag_expert.py:393-422`` expects routed tensors).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from . import collectives, symm

_v, _i = ctypes.c_void_p, ctypes.c_int
_native.declare("dd_moe_peer", symm._TEAM + [_i, _v, _v, _v, _v, _v, _i, _i, _i, _i, _i, ctypes.POINTER(_i), _v])


def usable(x: torch.Tensor, ranks, e_local: int, capacity: int) -> bool:
    d = x.shape[-1]
    P = len(ranks)
    return (x.is_cuda and x.dtype == torch.bfloat16 and d % 8 == 0 and 1 < P <= 8 and collectives.available(ranks)
            and symm.heap_ready() and e_local * P * capacity * d * 2 <= symm.heap().staging_bytes)


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _run(mode, ranks, x, ids, slot, w, out, tokens, k, El, C, d):
    collectives._launch("dd_moe_peer", symm.heap(), list(ranks), mode, x.data_ptr(), ids.data_ptr(), slot.data_ptr(),
                        _ptr(w), _ptr(out), tokens, k, El, C, d)


def _stage(ranks, El, C, d):
    P = len(ranks)
    return symm.heap().staging_tensor(El * P * C * d * 2, torch.bfloat16)


class PeerDispatchFn(torch.autograd.Function):
    """x [T, d] -> [El, P * C, d]: rows of the local experts from all source GPUs."""

    @staticmethod
    def forward(ctx, x, ids, slot, ranks, El, C, k):
        T, d = x.shape
        xc = x.contiguous()
        stage = _stage(ranks, El, C, d)
        stage.zero_()                                   # unused capacity slots read as zero
        _run(0, ranks, xc, ids, slot, None, None, T, k, El, C, d)
        ctx.save_for_backward(ids, slot)
        ctx.cfg = (tuple(ranks), El, C, k, T, d)
        return stage.clone().view(El, len(ranks) * C, d)

    @staticmethod
    def backward(ctx, g):
        ids, slot = ctx.saved_tensors
        ranks, El, C, k, T, d = ctx.cfg
        stage = _stage(ranks, El, C, d)
        stage.copy_(g.reshape(-1))
        dx = torch.empty(T, d, dtype=g.dtype, device=g.device)
        _run(1, ranks, dx, ids, slot, None, None, T, k, El, C, d)
        return dx, None, None, None, None, None, None


class PeerCombineFn(torch.autograd.Function):
    """buf [El, P * C, d] (outputs of the local experts), w [T, k] -> y [T, d]."""

    @staticmethod
    def forward(ctx, buf, w, ids, slot, ranks, T, k, C):
        El, _, d = buf.shape
        bufc, wc = buf.contiguous(), w.reshape(-1).float().contiguous()
        stage = _stage(ranks, El, C, d)
        stage.copy_(bufc.reshape(-1))
        y = torch.empty(T, d, dtype=buf.dtype, device=buf.device)
        _run(1, ranks, y, ids, slot, wc, None, T, k, El, C, d)
        ctx.save_for_backward(bufc, wc, ids, slot)
        ctx.cfg = (tuple(ranks), El, C, k, T, d, w.shape, w.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        buf, w, ids, slot = ctx.saved_tensors
        ranks, El, C, k, T, d, wshape, wdtype = ctx.cfg
        dyc = dy.contiguous()
        stage = _stage(ranks, El, C, d)
        # router-weight gradients: <dy[t], expert output row>, rows read from their owners
        stage.copy_(buf.reshape(-1))
        dots = torch.empty(T * k, dtype=torch.float32, device=dy.device)
        _run(2, ranks, dyc, ids, slot, None, dots, T, k, El, C, d)
        # gradient of the expert outputs: w * dy scattered to the owners
        stage.zero_()
        _run(0, ranks, dyc, ids, slot, w, None, T, k, El, C, d)
        dbuf = stage.clone().view(buf.shape)
        return dbuf, dots.reshape(wshape).to(wdtype), None, None, None, None, None, None


def dispatch(x, ids, slot, ranks, e_local, capacity, k):
    return PeerDispatchFn.apply(x, ids, slot, tuple(ranks), e_local, capacity, k)


def combine(buf, weights, ids, slot, ranks, tokens, k, capacity):
    return PeerCombineFn.apply(buf, weights, ids, slot, tuple(ranks), tokens, k, capacity)
