"""Lets a worker that holds no loss value still call ``.backward()``
(``src/distdl/functional/zero_volume_corrector.py:7-87``)."""
import torch

from ..utilities.torch import zero_volume_tensor


class ZeroVolumeCorrectorFunction(torch.autograd.Function):
    """Forward: a zero-volume tensor becomes a scalar 0 that requires grad;
    anything else passes through.  Backward: the scalar's gradient becomes a
    zero-volume tensor again, so upstream adjoints see "nothing here"."""

    @staticmethod
    def forward(ctx, input):
        ctx.was_empty = input.numel() == 0
        ctx.in_shape = tuple(input.shape)
        ctx.dtype, ctx.device = input.dtype, input.device
        if ctx.was_empty:
            return torch.zeros((), dtype=input.dtype, device=input.device, requires_grad=True)
        return input.clone()

    @staticmethod
    def backward(ctx, grad_output):
        if ctx.was_empty:
            b = ctx.in_shape[0] if len(ctx.in_shape) == 2 else None
            return zero_volume_tensor(b, dtype=ctx.dtype, device=ctx.device)
        return grad_output.clone()
