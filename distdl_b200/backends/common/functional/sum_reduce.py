"""SumReduce: members of every team add their tensors onto the team's root.
Adjoint: broadcast of the root's gradient.
(``src/distdl/backends/mpi_numpy/functional/sum_reduce.py:104-117``, ``:197-215``.)"""
from __future__ import annotations

import torch

from ._base import TransportBound, empty_output
from .broadcast import _ordered_roles


class SumReduceFunction(TransportBound, torch.autograd.Function):
    # P_send: the team this worker contributes in; P_recv: the team it is the root of.
    @staticmethod
    def forward(ctx, input, P_send, P_recv, preserve_batch, input_tensor_structure, output_tensor_structure):
        cls = ctx._forward_cls
        t = cls.transport()
        device = input.device
        ctx.P_send, ctx.P_recv = P_send, P_recv
        ctx.preserve_batch = preserve_batch
        ctx.input_tensor_structure = input_tensor_structure
        ctx.output_tensor_structure = output_tensor_structure
        ctx.device = device
        output = empty_output(input, preserve_batch, device)
        same = P_send.active and P_recv.active and P_send.ranks == P_recv.ranks
        # roles: in P_recv I am the root, in P_send a member
        for role, P in _ordered_roles(P_recv, P_send):
            if role == "root":
                if same:
                    contrib = input.detach()
                else:
                    contrib = torch.zeros(tuple(output_tensor_structure.shape), dtype=output_tensor_structure.dtype,
                                          device=device)
                output = t.reduce(contrib, list(P.ranks), 0)
            else:
                t.reduce(input.detach(), list(P.ranks), 0)
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
        for role, P in _ordered_roles(P_recv, P_send):
            if role == "root":
                t.broadcast(grad_output.detach(), list(P.ranks), 0)
                if same:
                    grad_input = grad_output.clone()
            else:
                buf = torch.empty(tuple(its.shape), dtype=its.dtype, device=device)
                t.broadcast(buf, list(P.ranks), 0)
                grad_input = buf
        return grad_input, None, None, None, None, None
