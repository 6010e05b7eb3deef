"""AllGather along one tensor axis inside a team; adjoint = reduce-scatter.
Uneven shards follow the balanced rule (first ``n % P`` members hold one more).
(``src/distdl/backends/nccl_cupy/functional/all_gather.py:86-139``, ``:220-227``.)"""
from __future__ import annotations

import torch

from ._base import TransportBound, scaled


def member_extents(n, P):
    return [n // P + (1 if i < n % P else 0) for i in range(P)]


class AllGatherFunction(TransportBound, torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, P_allgather, input_tensor_structure, output_tensor_structure, axes, scale_backward):
        cls = ctx._forward_cls
        ctx.P_allgather = P_allgather
        ctx.axes = axes
        ctx.scale_backward = scale_backward
        ctx.input_tensor_structure = input_tensor_structure
        # A parameter whose gradient is accumulated elsewhere (unsharded accumulator of the
        # optimizer) produces no gradient for the gathered tensor: its adjoint is then skipped
        # instead of reduce-scattering zeros.  Every member of the team sets the accumulator
        # up or none does, so the decision is the same everywhere.
        ctx.skip_without_grad = getattr(input, "full_grad_view", None) is not None
        ctx.set_materialize_grads(False)
        ctx.out_meta = None
        if not P_allgather.active:
            return input.clone()
        axis = int(axes[0])
        P = P_allgather.size
        n = int(output_tensor_structure.shape[axis])
        ext = member_extents(n, P)
        if int(input.shape[axis]) != ext[P_allgather.rank]:
            raise ValueError(f"AllGather: local extent {input.shape[axis]} along axis {axis} does not follow the "
                             f"balanced split of {n} over {P} workers")
        ctx.extents = ext
        # a parameter with an fp32 gradient accumulator (set by the optimizer) gets its
        # reduce-scattered gradient added there directly in backward
        ctx.grad_acc = getattr(input, "main_grad_view", None)
        shapes = None
        if len(set(ext)) > 1:
            shapes = []
            for e in ext:
                s = list(input.shape)
                s[axis] = e
                shapes.append(s)
        if axis == 0 and shapes is None:
            # equal shards along the leading axis: the stacked result *is* the concatenation
            stacked = cls.transport().allgather_stacked(input.detach(), list(P_allgather.ranks))
            out = stacked.reshape((-1,) + tuple(input.shape[1:]))
        else:
            parts = cls.transport().allgather(input.detach(), list(P_allgather.ranks), shapes)
            out = torch.cat(parts, dim=axis)
        out.requires_grad_(bool(output_tensor_structure.requires_grad) and out.is_floating_point())
        ctx.out_meta = (tuple(out.shape), out.dtype, out.device)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        cls = ctx._forward_cls
        P = ctx.P_allgather
        if grad_output is None:
            if ctx.skip_without_grad or not P.active or ctx.out_meta is None:
                return None, None, None, None, None, None
            shape, dtype, device = ctx.out_meta
            grad_output = torch.zeros(shape, dtype=dtype, device=device)
        if not P.active:
            return grad_output.clone(), None, None, None, None, None
        axis = int(ctx.axes[0])
        g = scaled(grad_output, ctx.scale_backward).detach()
        if axis == 0 and len(set(ctx.extents)) == 1:
            t = cls.transport()
            if ctx.grad_acc is not None and hasattr(t, "reduce_scatter_accumulate") and grad_output.is_cuda:
                gs = grad_output.contiguous().reshape(P.size, -1)
                scale = 1.0 if ctx.scale_backward is None else 1.0 / float(ctx.scale_backward)
                if t.reduce_scatter_accumulate(gs, ctx.grad_acc, list(P.ranks), scale):
                    return None, None, None, None, None, None
            stacked = g.contiguous().reshape((P.size, ctx.extents[0]) + tuple(g.shape[1:]))
            out = t.reduce_scatter_stacked(stacked, list(P.ranks))
        else:
            chunks = list(torch.split(g, ctx.extents, dim=axis))
            out = cls.transport().reduce_scatter(chunks, list(P.ranks))
        return out, None, None, None, None, None
