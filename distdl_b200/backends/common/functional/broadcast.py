"""Broadcast: the root of every team sends its tensor to the team's members.
Adjoint: sum-reduction of the members' gradients onto the root.
(``src/distdl/backends/mpi_numpy/functional/broadcast.py:110-126``, ``:194-209``.)"""
from __future__ import annotations

import torch

from ._base import TransportBound, empty_output, scaled


def _ordered_roles(P_send, P_recv):
    """The (role, team) pairs of this worker, lowest root first on every worker
    so that blocking transports cannot wait on each other in a cycle."""
    roles = []
    if P_send.active:
        roles.append(("root", P_send))
    if P_recv.active and not (P_send.active and P_recv.ranks == P_send.ranks):
        roles.append(("member", P_recv))
    roles.sort(key=lambda r: r[1].ranks[0])
    return roles


class BroadcastFunction(TransportBound, torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, P_send, P_recv, preserve_batch, input_tensor_structure, output_tensor_structure,
                scale_backward):
        cls = ctx._forward_cls
        t = cls.transport()
        device = input.device
        ctx.P_send, ctx.P_recv = P_send, P_recv
        ctx.preserve_batch = preserve_batch
        ctx.input_tensor_structure = input_tensor_structure
        ctx.output_tensor_structure = output_tensor_structure
        ctx.scale_backward = scale_backward
        ctx.device = device
        output = empty_output(input, preserve_batch, device)
        same = P_send.active and P_recv.active and P_send.ranks == P_recv.ranks
        for role, P in _ordered_roles(P_send, P_recv):
            if role == "root":
                t.broadcast(input.detach(), list(P.ranks), 0)
                if same:
                    output = input.clone()
            else:
                buf = torch.empty(tuple(output_tensor_structure.shape), dtype=output_tensor_structure.dtype,
                                  device=device)
                t.broadcast(buf, list(P.ranks), 0)
                output = buf
        if P_recv.active:
            output.requires_grad_(bool(output_tensor_structure.requires_grad) and output.is_floating_point())
        return output

    @staticmethod
    def backward(ctx, grad_output):
        cls = ctx._forward_cls
        t = cls.transport()
        P_send, P_recv = ctx.P_send, ctx.P_recv
        device = ctx.device
        its = ctx.input_tensor_structure
        grad_input = empty_output(grad_output, ctx.preserve_batch, device)
        same = P_send.active and P_recv.active and P_send.ranks == P_recv.ranks
        for role, P in _ordered_roles(P_send, P_recv):
            if role == "root":
                if same:
                    contrib = scaled(grad_output, ctx.scale_backward)
                else:
                    # the root holds no copy of the output: it contributes zero
                    contrib = torch.zeros(tuple(its.shape), dtype=its.dtype, device=device)
                grad_input = t.reduce(contrib, list(P.ranks), 0)
            else:
                t.reduce(scaled(grad_output, ctx.scale_backward), list(P.ranks), 0)
        return grad_input, None, None, None, None, None, None
