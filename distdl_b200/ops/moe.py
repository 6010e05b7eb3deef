"""Mixture-of-experts token routing ops (slot assignment, permuted scatter,
weighted gather) with autograd; CUDA kernels in ``csrc/moe.cu``.  New relative to
the reference (its expert layers expect already-routed ``[expert, capacity,
...]`` tensors, ``src/distdl/nn/linear_ag_expert.py:393-422``)."""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import ptr, stream_ptr, use_native

_v, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_native.declare("dd_moe_assign", [_v, _i, _i, _i, _v, _v, _v])
_native.declare("dd_moe_chunks", [_i])


def _counters(items: int, E: int, device):
    """Scratch of the slot assignment: [0, E) receives the pairs per expert, the rest holds the
    per-chunk histograms."""
    chunks = _native.lib().dd_moe_chunks(int(items))
    return torch.empty((chunks + 1) * E, dtype=torch.int32, device=device)
_native.declare("dd_moe_scatter_rows", [_v, _v, _v, _v, _v, _i, _i, _i, _i, _v])
_native.declare("dd_moe_gather_rows", [_v, _v, _v, _v, _v, _i, _i, _i, _i, _v])
_native.declare("dd_moe_pair_dot", [_v, _v, _v, _v, _v, _i, _i, _i, _i, _v])


_native.declare("dd_moe_router_fwd", [_v, _i, _i, _i, _i, _i, _v, _v, _v, _v, _v, _v])
_native.declare("dd_moe_router_bwd", [_v, _i, _i, _i, _i, _v, _v, _v, _v, _v, _v])


class _RouterFn(torch.autograd.Function):
    """Softmax over the experts, top-k, renormalised weights and the column sums of the probabilities
    in one kernel, the slots (arrival order = pair index, so overflow drops the same pairs in every
    run) in a second one; one more kernel for the backward pass."""

    @staticmethod
    def forward(ctx, logits, E, k, capacity):
        T, ld = logits.shape
        dev = logits.device
        ids = torch.empty(T * k, dtype=torch.int32, device=dev)
        w = torch.empty(T, k, dtype=torch.float32, device=dev)
        slot = torch.empty(T * k, dtype=torch.int32, device=dev)
        scratch = _counters(T, E, dev)
        counts = scratch[:E]
        prob_sum = torch.zeros(E, dtype=torch.float32, device=dev)
        _native.call("dd_moe_router_fwd", logits.data_ptr(), ld, T, E, k, capacity, ids.data_ptr(), w.data_ptr(),
                     slot.data_ptr(), scratch.data_ptr(), prob_sum.data_ptr(), stream_ptr())
        ctx.save_for_backward(logits, ids, w)
        ctx.cfg = (E, k)
        ctx.mark_non_differentiable(ids, slot, counts)
        ctx.set_materialize_grads(False)
        return w, prob_sum, ids, slot, counts

    @staticmethod
    def backward(ctx, dw, dprob, _dids, _dslot, _dcounts):
        logits, ids, w = ctx.saved_tensors
        E, k = ctx.cfg
        T, ld = logits.shape
        dlogits = torch.empty_like(logits)
        dwc = None if dw is None else dw.float().contiguous()
        dpc = None if dprob is None else dprob.float().contiguous()
        _native.call("dd_moe_router_bwd", logits.data_ptr(), ld, T, E, k, ids.data_ptr(), w.data_ptr(), ptr(dwc),
                     ptr(dpc), dlogits.data_ptr(), stream_ptr())
        return dlogits, None, None, None


def route(logits: torch.Tensor, num_experts: int, k: int, capacity: int):
    """Top-k routing of ``logits [tokens, >= num_experts]`` (extra columns are padding).

    Returns ``(weights [tokens, k] fp32, prob_sum [E] fp32, ids [tokens * k] int32, slot
    [tokens * k] int32, counts [E] int32)``: the renormalised softmax weights of the chosen
    experts, the sum over tokens of the softmax probabilities (for the load-balancing loss), the
    chosen experts, each pair's slot in its expert's capacity buffer (-1 = dropped) and the number
    of pairs routed to every expert.  ``weights`` and ``prob_sum`` carry gradients back to
    ``logits``."""
    E = num_experts
    if use_native(logits) and logits.dtype == torch.bfloat16 and E <= 64 and k <= 8 and logits.is_contiguous():
        return _RouterFn.apply(logits, E, k, capacity)
    probs = torch.softmax(logits[:, :E].float(), dim=-1)
    topw, topi = probs.topk(k, dim=-1)
    topw = topw / topw.sum(-1, keepdim=True)
    ids = topi.to(torch.int32).reshape(-1).contiguous()
    slot, counts = assign_slots(ids, E, capacity)
    return topw, probs.sum(0), ids, slot, counts


def assign_slots(ids: torch.Tensor, num_experts: int, capacity: int):
    """ids [pairs] int32 -> (slot [pairs] int32 with -1 for dropped pairs, counts [E] int32)."""
    flat = ids.reshape(-1).to(torch.int32).contiguous()
    if use_native(flat):
        scratch = _counters(flat.numel(), num_experts, flat.device)
        slot = torch.empty_like(flat)
        _native.call("dd_moe_assign", flat.data_ptr(), flat.numel(), num_experts, capacity, scratch.data_ptr(),
                     slot.data_ptr(), stream_ptr())
        return slot, scratch[:num_experts]
    onehot = torch.nn.functional.one_hot(flat.long(), num_experts)
    pos = (onehot.cumsum(0) - 1)[torch.arange(flat.numel()), flat.long()]
    slot = torch.where(pos < capacity, pos, torch.full_like(pos, -1)).to(torch.int32)
    return slot, onehot.sum(0).to(torch.int32)


def _scatter(src, ids, slot, w, E, C, k):
    d = src.shape[-1]
    dst = torch.zeros(E, C, d, dtype=src.dtype, device=src.device)
    if use_native(src) and src.dtype == torch.bfloat16 and d % 8 == 0:
        _native.call("dd_moe_scatter_rows", src.data_ptr(), ids.data_ptr(), slot.data_ptr(), ptr(w), dst.data_ptr(),
                     ids.numel(), k, C, d, stream_ptr())
        return dst
    keep = slot >= 0
    rows = src[torch.arange(ids.numel(), device=src.device) // k]
    if w is not None:
        rows = rows * w.reshape(-1, 1).to(rows.dtype)
    dst[ids[keep].long(), slot[keep].long()] = rows[keep]
    return dst


def _gather(src, ids, slot, w, tokens, k):
    E, C, d = src.shape
    if use_native(src) and src.dtype == torch.bfloat16 and d % 8 == 0:
        dst = torch.empty(tokens, d, dtype=src.dtype, device=src.device)
        _native.call("dd_moe_gather_rows", src.data_ptr(), ids.data_ptr(), slot.data_ptr(), ptr(w), dst.data_ptr(),
                     tokens, k, C, d, stream_ptr())
        return dst
    keep = (slot >= 0).reshape(tokens, k, 1)
    rows = src[ids.long().clamp(min=0), slot.long().clamp(min=0)].reshape(tokens, k, d).float()
    if w is not None:
        rows = rows * w.reshape(tokens, k, 1)
    return (rows * keep).sum(1).to(src.dtype)


def _pair_dot(a, b, ids, slot, k):
    E, C, d = b.shape
    n = ids.numel()
    if use_native(a) and a.dtype == torch.bfloat16 and d % 8 == 0:
        out = torch.empty(n, dtype=torch.float32, device=a.device)
        _native.call("dd_moe_pair_dot", a.data_ptr(), b.data_ptr(), ids.data_ptr(), slot.data_ptr(), out.data_ptr(),
                     n, k, C, d, stream_ptr())
        return out
    rows = b[ids.long().clamp(min=0), slot.long().clamp(min=0)].float()
    av = a[torch.arange(n, device=a.device) // k].float()
    return (rows * av).sum(-1) * (slot >= 0)


class DispatchFn(torch.autograd.Function):
    """x [T, d] -> per-expert capacity buffers [E, C, d] (unused slots zero)."""

    @staticmethod
    def forward(ctx, x, ids, slot, E, C, k):
        ctx.save_for_backward(ids, slot)
        ctx.cfg = (x.shape[0], k)
        return _scatter(x.contiguous(), ids, slot, None, E, C, k)

    @staticmethod
    def backward(ctx, g):
        ids, slot = ctx.saved_tensors
        T, k = ctx.cfg
        return _gather(g.contiguous(), ids, slot, None, T, k), None, None, None, None, None


class CombineFn(torch.autograd.Function):
    """y[t] = sum_c w[t, c] * buf[ids[t, c], slot[t, c]]."""

    @staticmethod
    def forward(ctx, buf, w, ids, slot, T, k):
        bufc, wc = buf.contiguous(), w.reshape(-1).float().contiguous()
        ctx.save_for_backward(bufc, wc, ids, slot)
        ctx.cfg = (T, k, w.shape, w.dtype)
        return _gather(bufc, ids, slot, wc, T, k)

    @staticmethod
    def backward(ctx, dy):
        buf, w, ids, slot = ctx.saved_tensors
        T, k, wshape, wdtype = ctx.cfg
        E, C, d = buf.shape
        dyc = dy.contiguous()
        dbuf = _scatter(dyc, ids, slot, w, E, C, k)
        dw = _pair_dot(dyc, buf, ids, slot, k).reshape(wshape).to(wdtype)
        return dbuf, dw, None, None, None, None


def dispatch(x, ids, slot, num_experts, capacity, k):
    return DispatchFn.apply(x, ids, slot, num_experts, capacity, k)


def combine(buf, weights, ids, slot, tokens, k):
    return CombineFn.apply(buf, weights, ids, slot, tokens, k)
