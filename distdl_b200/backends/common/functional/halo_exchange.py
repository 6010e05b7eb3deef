"""HaloExchange: neighbours on a Cartesian grid swap boundary slabs, one
dimension after another so that corners propagate.  Adjoint: dimensions in
reverse; ghost gradients travel back, are added into the bulk and cleared.
(``src/distdl/backends/mpi_numpy/functional/halo_exchange.py:46-72``, ``:110-138``.)

``slices[d] = (left_bulk, left_ghost, right_bulk, right_ghost)`` (nd-slices of
the local tensor), ``neighbor_ranks[d] = (left, right)`` as *world* ranks or
``PROC_NULL``."""
from __future__ import annotations

import torch

from ..world import PROC_NULL
from ._base import TransportBound


def _volume(sl):
    v = 1
    for s in sl:
        v *= max(0, s.stop - s.start)
    return v


def _shape(sl):
    return tuple(max(0, s.stop - s.start) for s in sl)


_plans = {}


def _box_plan(t, kind, x, P_x, slices, neighbor_ranks):
    """The one-kernel form of the exchange on transports that have it (device tensors on the
    native backend): all dimensions in one launch, one phase per dimension, faces packed into
    the neighbours' inboxes and unpacked (or added and cleared, for the adjoint) by the kernel."""
    maker = getattr(t, "box_plan", None)
    if maker is None or not (x.is_cuda or getattr(t, "box_plans_on_host", False)):
        return None
    key = (kind, id(t), tuple(int(r) for pair in neighbor_ranks for r in pair),
           tuple((s.start, s.stop) for per_dim in slices for box in per_dim for s in box))
    plan = _plans.get(key, False)
    if plan is not False:
        return plan
    phases = []
    dims = range(P_x.dim) if kind == "fill" else reversed(range(P_x.dim))
    for d in dims:
        lb, lg, rb, rg = slices[d]
        left, right = neighbor_ranks[d]
        ops = []
        for nbr, bulk, ghost in ((left, lb, lg), (right, rb, rg)):
            if nbr == PROC_NULL:
                continue
            if kind == "fill":
                if _volume(bulk):
                    ops.append(("send", nbr, "x", bulk, False))
                if _volume(ghost):
                    ops.append(("recv", nbr, "x", ghost, False))
            else:
                if _volume(ghost):
                    ops.append(("send", nbr, "x", ghost, True))      # ghosts leave and are cleared
                if _volume(bulk):
                    ops.append(("recv", nbr, "x", bulk, True))       # and are added to the owner's bulk
        phases.append(ops)
    plan = maker(phases, list(P_x.ranks))
    _plans[key] = plan
    return plan


def _staged(buffers, d, k, like, shape):
    """View ``k`` (0 / 1: left send / receive, 2 / 3: right send / receive) of the layer's staging
    buffers for dimension ``d`` if it can carry a message of ``shape`` for tensor ``like``."""
    if buffers is None or buffers[d] is None:
        return None
    b = buffers[d][k]
    if b is None or b.dtype != like.dtype or b.device != like.device or tuple(b.shape) != tuple(shape):
        return None
    return b


def _packed(buf, face):
    """The face as a contiguous message: packed into the staging view when there is one."""
    return face if buf is None else buf.copy_(face)


def fill_ghosts(t, x, P_x, slices, neighbor_ranks, buffers=None):
    """The exchange itself: a copy of ``x`` whose ghost regions hold the neighbours' bulk regions.
    On the transports that move whole messages (``recv_into``), the faces are packed into and
    received into the views that the layer obtained from its buffer manager."""
    out = x.detach().clone()
    plan = _box_plan(t, "fill", out, P_x, slices, neighbor_ranks)
    if plan is not None:
        plan.run(x=out)
        return out
    for d in range(P_x.dim):
        lb, lg, rb, rg = slices[d]
        left, right = neighbor_ranks[d]
        sends, recvs, targets = [], [], []
        staged = buffers if getattr(t, "recv_into", False) else None
        if left != PROC_NULL:
            if _volume(lb):
                sends.append((left, _packed(_staged(staged, d, 0, out, _shape(lb)), out[lb])))
            if _volume(lg):
                recvs.append((left, _shape(lg), out.dtype, _staged(staged, d, 1, out, _shape(lg))))
                targets.append(lg)
        if right != PROC_NULL:
            if _volume(rb):
                sends.append((right, _packed(_staged(staged, d, 2, out, _shape(rb)), out[rb])))
            if _volume(rg):
                recvs.append((right, _shape(rg), out.dtype, _staged(staged, d, 3, out, _shape(rg))))
                targets.append(rg)
        if staged is None:
            recvs = [r[:3] for r in recvs]
        got = t.exchange(sends, recvs, list(P_x.ranks))
        for sl, g in zip(targets, got):
            out[sl] = g.to(out.device)
    return out


def fold_ghosts(t, x, P_x, slices, neighbor_ranks, buffers=None):
    """The adjoint of :func:`fill_ghosts`: ghost regions travel to the neighbours they came from,
    are ADDED to the bulk regions there, and are cleared here.  The staging views swap roles: a
    ghost leaves through the view that received it, a bulk contribution arrives in the view that
    sent the bulk."""
    g = x.detach().clone()
    plan = _box_plan(t, "fold", g, P_x, slices, neighbor_ranks)
    if plan is not None:
        plan.run(x=g)
        return g
    for d in reversed(range(P_x.dim)):
        lb, lg, rb, rg = slices[d]
        left, right = neighbor_ranks[d]
        sends, recvs, targets = [], [], []
        staged = buffers if getattr(t, "recv_into", False) else None

        def leaving(k, sl):
            buf = _staged(staged, d, k, g, _shape(sl))
            return g[sl].clone() if buf is None else buf.copy_(g[sl])
        if left != PROC_NULL:
            if _volume(lg):
                sends.append((left, leaving(1, lg)))
            if _volume(lb):
                recvs.append((left, _shape(lb), g.dtype, _staged(staged, d, 0, g, _shape(lb))))
                targets.append(lb)
        if right != PROC_NULL:
            if _volume(rg):
                sends.append((right, leaving(3, rg)))
            if _volume(rb):
                recvs.append((right, _shape(rb), g.dtype, _staged(staged, d, 2, g, _shape(rb))))
                targets.append(rb)
        if staged is None:
            recvs = [r[:3] for r in recvs]
        got = t.exchange(sends, recvs, list(P_x.ranks))
        if left != PROC_NULL and _volume(lg):
            g[lg] = 0
        if right != PROC_NULL and _volume(rg):
            g[rg] = 0
        for sl, r in zip(targets, got):
            g[sl] += r.to(g.device)
    return g


class HaloExchangeFunction(TransportBound, torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, P_x, slices, buffers, neighbor_ranks):
        cls = ctx._forward_cls
        ctx.P_x, ctx.slices, ctx.neighbor_ranks = P_x, slices, neighbor_ranks
        if not P_x.active or P_x.size == 1:
            ctx.identity = True
            return input
        ctx.identity = False
        ctx.buffers = buffers
        out = fill_ghosts(cls.transport(), input, P_x, slices, neighbor_ranks, buffers)
        out.requires_grad_(input.requires_grad)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.identity:
            return grad_output, None, None, None, None
        cls = ctx._forward_cls
        g = fold_ghosts(cls.transport(), grad_output, ctx.P_x, ctx.slices, ctx.neighbor_ranks, ctx.buffers)
        return g, None, None, None, None


class HaloAccumulateFunction(TransportBound, torch.autograd.Function):
    """The halo exchange run backwards as a forward operation: every worker's ghost regions are
    added into the owning neighbours' bulk regions (and cleared).  Used where workers produce
    contributions to entries their neighbours own (transposed convolution).  Its adjoint is the
    plain exchange.  Same arguments as :class:`HaloExchangeFunction`."""

    @staticmethod
    def forward(ctx, input, P_x, slices, buffers, neighbor_ranks):
        cls = ctx._forward_cls
        ctx.P_x, ctx.slices, ctx.neighbor_ranks = P_x, slices, neighbor_ranks
        if not P_x.active or P_x.size == 1:
            ctx.identity = True
            return input
        ctx.identity = False
        ctx.buffers = buffers
        out = fold_ghosts(cls.transport(), input, P_x, slices, neighbor_ranks, buffers)
        out.requires_grad_(input.requires_grad)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.identity:
            return grad_output, None, None, None, None
        cls = ctx._forward_cls
        g = fill_ghosts(cls.transport(), grad_output, ctx.P_x, ctx.slices, ctx.neighbor_ranks, ctx.buffers)
        return g, None, None, None, None
