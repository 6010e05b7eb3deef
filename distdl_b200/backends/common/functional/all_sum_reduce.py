"""AllSumReduce: every member of the team ends with the sum; self-adjoint.
(``src/distdl/backends/mpi_numpy/functional/all_sum_reduce.py:77-85``, ``:128-136``.)"""
from __future__ import annotations

import torch

from ._base import TransportBound, scaled


class AllSumReduceFunction(TransportBound, torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, P_allreduce, input_tensor_structure, output_tensor_structure, scale_backward):
        cls = ctx._forward_cls
        ctx.P_allreduce = P_allreduce
        ctx.scale_backward = scale_backward
        if not P_allreduce.active:
            return input.clone()
        out = cls.transport().allreduce(input.detach(), list(P_allreduce.ranks))
        out.requires_grad_(bool(output_tensor_structure.requires_grad) and out.is_floating_point())
        return out

    @staticmethod
    def backward(ctx, grad_output):
        cls = ctx._forward_cls
        P = ctx.P_allreduce
        if not P.active:
            return grad_output.clone(), None, None, None, None
        g = cls.transport().allreduce(scaled(grad_output, ctx.scale_backward).detach(), list(P.ranks))
        return g, None, None, None, None
