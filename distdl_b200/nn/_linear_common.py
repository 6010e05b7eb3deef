"""Helpers shared by the tensor-parallel linear / expert / embedding layers:
derived partitions, serial <-> parallel weight re-layouts (fused QKV with or
without grouped-query heads, GEGLU / SwiGLU halves), prefetch streams.

Layout convention of a fused projection that is split over ``M`` tensor-parallel
workers along its output features: worker ``p`` stores the blocks
``[var_0(p) | var_1(p) | ...]`` ("parallel" layout, ``(p v h)``); a serial
checkpoint stores ``[var_0(all p) | var_1(all p) | ...]`` (``(v p h)``).  The
reference performs the same conversions with einops patterns
(``src/distdl/nn/linear_ag.py:275-354``).
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..utilities.slicing import compute_subshape, worker_layout


def derived_partition(P, index, shape):
    """Sub-team of Cartesian partition ``P`` selected by the nd ``index`` (tuple
    of slices into ``worker_layout(P.shape)``), arranged with grid ``shape``."""
    workers = worker_layout(P.shape)[tuple(index)].reshape(-1).tolist()
    base = P.create_partition_inclusive(workers)
    return base.create_cartesian_topology_partition(shape)


def root_partition(P):
    """1-worker Cartesian partition (all dims 1) holding rank 0 of ``P``."""
    return P.create_partition_inclusive([0]).create_cartesian_topology_partition([1] * P.dim)


def split_sizes(n, P):
    return [int(compute_subshape(P, i, [n])[0]) for i in range(P)]


def var_blocks(out_features, num_gpu, num_heads=None, num_heads_kv=None, num_vars=3, geglu=False):
    """``blocks[p][v]`` = width of variable ``v`` on tensor-parallel worker ``p``."""
    if num_heads is not None and num_heads_kv is not None:
        head = out_features // (num_heads + 2 * num_heads_kv)
        hq, hkv = split_sizes(num_heads, num_gpu), split_sizes(num_heads_kv, num_gpu)
        return [[hq[p] * head, hkv[p] * head, hkv[p] * head] for p in range(num_gpu)]
    if num_heads is not None:
        head = out_features // num_vars // num_heads
        hq = split_sizes(num_heads, num_gpu)
        return [[hq[p] * head] * num_vars for p in range(num_gpu)]
    if geglu:
        half = split_sizes(out_features // 2, num_gpu)
        return [[half[p], half[p]] for p in range(num_gpu)]
    return None


def relayout(t, axis, blocks, to_serial):
    """Re-orders the blocks of ``t`` along ``axis`` between the parallel
    ``(p v)`` and the serial ``(v p)`` order."""
    if blocks is None:
        return t
    P, V = len(blocks), len(blocks[0])
    order_par = [(p, v) for p in range(P) for v in range(V)]
    order_ser = [(p, v) for v in range(V) for p in range(P)]
    src_order, dst_order = (order_par, order_ser) if to_serial else (order_ser, order_par)
    sizes = [blocks[p][v] for p, v in src_order]
    pieces = dict(zip(src_order, torch.split(t, sizes, dim=axis)))
    return torch.cat([pieces[k] for k in dst_order], dim=axis)


def local_out_features(out_features, num_gpu, index, num_heads=None, num_heads_kv=None, num_vars=3, geglu=False):
    """Output features stored on tensor-parallel worker ``index`` (a whole number
    of heads / an equal share of each GEGLU half when those are given)."""
    blocks = var_blocks(out_features, num_gpu, num_heads, num_heads_kv, num_vars, geglu)
    if blocks is None:
        return int(compute_subshape(num_gpu, index, [out_features])[0])
    return int(sum(blocks[index]))


def deliver_grad(param, g):
    """Adds the gradient shard ``g`` to ``param``: into the optimizer's fp32
    accumulator when the parameter has one (``main_grad_view``), else into
    ``param.grad``.  Used where a layer produces a parameter gradient outside of
    autograd (the deferred reduce-scatter of ZeRO-1 mode)."""
    acc = getattr(param, "main_grad_view", None)
    if acc is not None:
        from ..ops.optim import accumulate_f32_
        accumulate_f32_(acc, g)
    else:
        g = g.to(param.dtype)          # (an fp32 accumulation of a bf16 parameter's gradient)
        param.grad = g if param.grad is None else param.grad + g


def direct_main_grad(param, gather, shape):
    """An fp32 gradient buffer, viewed with the gathered ``shape``, into which the
    weight-gradient GEMM of a ZeRO layer may accumulate directly, or None.

    * the all-gather ``gather`` of ``param`` is the identity (one worker along the
      gathered dimension): the optimizer's accumulator of the shard itself;
    * otherwise, when the optimizer set one up (``param.full_grad_view``): the
      UNSHARDED accumulator of this step, which the optimizer reduce-scatters once,
      at the step, instead of after every micro-batch.
    Autograd then sees no gradient for the gathered weight, so the per-micro-batch
    reduce-scatter adjoint of the all-gather does not run."""
    acc = getattr(param, "main_grad_view", None)
    if acc is None or not param.is_cuda or os.environ.get("DISTDL_DIRECT_MAIN_GRAD", "1") == "0":
        return None
    if gather.scale_backward is not None:
        return None
    axis = gather.axes_all_gather[0]
    if int(gather.P_x.shape[axis]) == 1:
        return acc.view(shape)
    full = getattr(param, "full_grad_view", None)
    if full is not None and full.numel() == int(np.prod(shape)):
        return full.view(shape)
    return None


def reduce_scatter_grad(rs, full_grad, param, scale_backward=None):
    """Reduce-scatters the gradient accumulated on a gathered parameter and
    delivers the slice to ``param`` (fused into the fp32 accumulator when the
    transport can)."""
    acc = getattr(param, "main_grad_view", None)
    scale = 1.0 if scale_backward is None else 1.0 / float(scale_backward)
    if acc is not None and rs.accumulate_into(full_grad, acc, scale):
        return
    g = full_grad if scale_backward is None else full_grad / scale_backward
    deliver_grad(param, rs(g))


class KeptBufferGuard:
    """Detects a kept (``auto_clear_buffer=False``) gathered buffer that has gone stale: the
    shard parameters were updated in place (an optimizer step) without
    ``clear_weight_buffer()`` in between.  The stale copy is dropped and re-gathered, with a
    one-time warning, because the gradients accumulated on it were never delivered."""

    _warned = False

    def __init__(self):
        self.versions = None

    def remember(self, *params):
        self.versions = tuple(p._version for p in params if p is not None)

    def stale(self, *params):
        if self.versions is None:
            return False
        now = tuple(p._version for p in params if p is not None)
        if now == self.versions:
            return False
        if not KeptBufferGuard._warned:
            KeptBufferGuard._warned = True
            import warnings
            warnings.warn("a ZeRO layer with auto_clear_buffer=False saw its parameters change while a gathered "
                          "copy was kept: call clear_weight_buffer() (or model.release_gathered()) before the "
                          "optimizer step; the stale copy is re-gathered and its pending gradients are dropped")
        return True


class PrefetchStream:
    """Weight prefetch of a layer.  ``run(fn)`` executes ``fn`` (the gathers) on the current
    stream; gathers that need no handshake with other GPUs (parameter shards read in place
    from the optimizer's peer-mapped buffer) are moved to the device's side stream inside
    ``fn`` and are not waited for until ``wait()``, so a prefetch issued early overlaps the
    compute that follows it.  ``wait()`` waits for THIS layer's gathers only (an event
    recorded right after them), not for prefetches of other layers queued later on the same
    side stream.  Everything else stays ordered on the current stream."""

    def __init__(self, device):
        self.cuda = torch.cuda.is_available() and torch.device(device).type == "cuda"
        self._event = None

    def run(self, fn):
        if not self.cuda:
            return fn()
        from ..utilities import streams
        with streams.deferred():
            out = fn()
        side = streams.side_stream()
        if side is not None:
            self._event = torch.cuda.Event()
            self._event.record(side)
        return out

    def wait(self):
        if self.cuda and self._event is not None:
            torch.cuda.current_stream().wait_event(self._event)
            self._event = None
