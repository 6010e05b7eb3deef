"""Repartition: generalised all-to-all between two Cartesian decompositions of
the same global tensor.  Adjoint: the reverse repartition.
(``src/distdl/backends/nccl_cupy/functional/repartition.py:116-205``, ``:282-343``.)

Each overlap entry is ``(slices, shape, partner)`` with ``partner`` a world
rank, ``"self"`` for the locally copied overlap, or all ``None`` when the two
sub-tensors do not intersect.  Whether the result needs a gradient is agreed
once at set-up (the reference broadcasts that flag from the host on every
call)."""
from __future__ import annotations

import numpy as np
import torch

from ._base import TransportBound, empty_output


_plans = {}


def _box_plan(transport, send_overlaps, recv_overlaps, team):
    """The one-kernel form on transports that have it: every overlap rectangle goes straight from
    the source tensor into the partner's inbox and from there into its place in the output."""
    maker = getattr(transport, "box_plan", None)
    if maker is None or team is None:
        return None

    def sig(overlaps):
        return tuple((None if sl is None else tuple((s.start, s.stop) for s in sl), str(p)) for sl, _, p in overlaps)
    key = (id(transport), sig(send_overlaps), sig(recv_overlaps), tuple(team))
    plan = _plans.get(key, False)
    if plan is not False:
        return plan
    ops = []
    self_src = next((sl for sl, _, p in send_overlaps if p == "self"), None)
    for sl, sh, partner in send_overlaps:
        if sl is not None and partner != "self":
            ops.append(("send", partner, "src", sl, False))
    for sl, sh, partner in recv_overlaps:
        if sl is None:
            continue
        if partner == "self":
            ops.append(("copy", "src", self_src, "out", sl))
        else:
            ops.append(("recv", partner, "out", sl, False))
    plan = maker([ops], list(team))
    _plans[key] = plan
    return plan


def _fits(buf, like_dtype, device, shape):
    return (buf is not None and buf.dtype == like_dtype and buf.device == torch.device(device)
            and tuple(buf.shape) == tuple(int(v) for v in shape))


def _move(transport, src_tensor, out_shape, out_dtype, send_overlaps, recv_overlaps, device, team=None,
          send_buffers=None, recv_buffers=None):
    """``send_buffers`` / ``recv_buffers``: the layer's staging views, aligned with the two overlap lists;
    transports that move whole messages pack into them and receive into them."""
    if (src_tensor.is_cuda or (out_shape is not None and torch.device(device).type == "cuda")
            or getattr(transport, "box_plans_on_host", False)):
        plan = _box_plan(transport, send_overlaps, recv_overlaps, team)
        if plan is not None:
            if send_overlaps and src_tensor.dtype != out_dtype:
                src_tensor = src_tensor.to(out_dtype)
            out = None
            if out_shape is not None:
                shape = tuple(int(s) for s in out_shape)
                covered = sum(int(np.prod([int(v) for v in sh])) for sl, sh, _ in recv_overlaps if sl is not None)
                alloc = torch.empty if covered == int(np.prod(shape)) else torch.zeros
                out = alloc(shape, dtype=out_dtype, device=device)
            tensors = {}
            if send_overlaps:
                tensors["src"] = src_tensor
            if out is not None:
                tensors["out"] = out
            plan.run(**tensors)
            return out
    staged = getattr(transport, "recv_into", False)
    sends, recvs = [], []
    for i, (sl, sh, partner) in enumerate(send_overlaps):
        if sl is None or partner == "self":
            continue
        buf = send_buffers[i] if staged and send_buffers is not None and i < len(send_buffers) else None
        piece = src_tensor[sl]
        fits = _fits(buf, src_tensor.dtype, src_tensor.device, piece.shape)
        sends.append((partner, buf.copy_(piece) if fits else piece))
    for i, (sl, sh, partner) in enumerate(recv_overlaps):
        if sl is None or partner == "self":
            continue
        buf = recv_buffers[i] if staged and recv_buffers is not None and i < len(recv_buffers) else None
        recvs.append((partner, sh, out_dtype, buf) if _fits(buf, out_dtype, device, sh) else (partner, sh, out_dtype))
    got = transport.exchange(sends, recvs, team)
    out = None
    if out_shape is not None:
        out = torch.zeros(tuple(int(s) for s in out_shape), dtype=out_dtype, device=device)
        k = 0
        for sl, sh, partner in recv_overlaps:
            if sl is None:
                continue
            if partner == "self":
                src_sl = next(s for s, _, p in send_overlaps if p == "self")
                out[sl] = src_tensor[src_sl]
            else:
                out[sl] = got[k].to(device)
                k += 1
    return out


class RepartitionFunction(TransportBound, torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, P_union, x_global_structure, x_local_structure, y_local_structure, P_x,
                P_x_to_y_overlaps, P_x_to_y_buffers, P_y, P_y_to_x_overlaps, P_y_to_x_buffers, preserve_batch):
        cls = ctx._forward_cls
        device = input.device
        ctx.args = (P_union, x_global_structure, x_local_structure, y_local_structure, P_x, P_x_to_y_overlaps,
                    P_y, P_y_to_x_overlaps, preserve_batch)
        ctx.buffers = (P_x_to_y_buffers, P_y_to_x_buffers)
        ctx.device = device
        if not P_union.active:
            return empty_output(input, preserve_batch, device)
        sends = P_x_to_y_overlaps if P_x.active else []
        recvs = P_y_to_x_overlaps if P_y.active else []
        out_shape = y_local_structure.shape if P_y.active else None
        out = _move(cls.transport(), input.detach(), out_shape, x_global_structure.dtype, sends, recvs, device,
                    list(P_union.ranks), P_x_to_y_buffers if P_x.active else None,
                    P_y_to_x_buffers if P_y.active else None)
        if out is None:
            b = input.shape[0] if (preserve_batch and input.dim() > 0) else None
            from ....utilities.torch import zero_volume_tensor
            out = zero_volume_tensor(b, dtype=x_global_structure.dtype, device=device)
        out.requires_grad_(bool(x_global_structure.requires_grad) and out.is_floating_point())
        return out

    @staticmethod
    def backward(ctx, grad_output):
        cls = ctx._forward_cls
        (P_union, x_global_structure, x_local_structure, y_local_structure, P_x, P_x_to_y_overlaps, P_y,
         P_y_to_x_overlaps, preserve_batch) = ctx.args
        device = ctx.device
        none = (None,) * 11
        if not P_union.active:
            return (empty_output(grad_output, preserve_batch, device),) + none
        sends = P_y_to_x_overlaps if P_y.active else []
        recvs = P_x_to_y_overlaps if P_x.active else []
        out_shape = x_local_structure.shape if P_x.active else None
        # the adjoint sends what the forward pass received and receives what it sent: the views swap roles
        g = _move(cls.transport(), grad_output.detach(), out_shape, x_global_structure.dtype, sends, recvs, device,
                  list(P_union.ranks), ctx.buffers[1] if P_y.active else None, ctx.buffers[0] if P_x.active else None)
        if g is None:
            from ....utilities.torch import zero_volume_tensor
            b = grad_output.shape[0] if (preserve_batch and grad_output.dim() > 0) else None
            g = zero_volume_tensor(b, dtype=x_global_structure.dtype, device=device)
        return (g,) + none
