"""ReduceScatter along one tensor axis inside a team; adjoint = all-gather.
(``src/distdl/backends/nccl_cupy/functional/reduce_scatter.py:83-136``, ``:188-194``.)"""
from __future__ import annotations

import torch

from ._base import TransportBound
from .all_gather import member_extents


class ReduceScatterFunction(TransportBound, torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, P_reducescatter, input_tensor_structure, output_tensor_structure, axes):
        cls = ctx._forward_cls
        ctx.P_reducescatter = P_reducescatter
        ctx.axes = axes
        if not P_reducescatter.active:
            return input.clone()
        axis = int(axes[0])
        P = P_reducescatter.size
        ext = member_extents(int(input.shape[axis]), P)
        ctx.extents = ext
        chunks = list(torch.split(input.detach(), ext, dim=axis))
        out = cls.transport().reduce_scatter(chunks, list(P_reducescatter.ranks))
        out.requires_grad_(bool(output_tensor_structure.requires_grad) and out.is_floating_point())
        return out

    @staticmethod
    def backward(ctx, grad_output):
        cls = ctx._forward_cls
        P = ctx.P_reducescatter
        if not P.active:
            return grad_output.clone(), None, None, None, None
        axis = int(ctx.axes[0])
        ext = ctx.extents
        shapes = None
        if len(set(ext)) > 1:
            shapes = []
            for e in ext:
                s = list(grad_output.shape)
                s[axis] = e
                shapes.append(s)
        parts = cls.transport().allgather(grad_output.detach(), list(P.ranks), shapes)
        return torch.cat(parts, dim=axis), None, None, None, None
