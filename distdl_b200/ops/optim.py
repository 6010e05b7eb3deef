"""Fused AdamW step and sum-of-squares kernels on flat fp32 buffers."""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, stream_ptr, use_native


def adamw_step_(master, m, v, grad, param_bf16, *, lr, beta1, beta2, eps, weight_decay, step,
                grad_scale_tensor=None, grad_scale=1.0, zero_grad=True):
    """In-place AdamW on flat fp32 ``master``/``m``/``v`` with fp32 ``grad``;
    refreshes the bf16 working copy and clears the gradient in the same pass."""
    n = master.numel()
    if n == 0:
        return
    if use_native(master):
        _native.call("dd_adamw", master.data_ptr(), m.data_ptr(), v.data_ptr(), grad.data_ptr(), ptr(param_bf16), n,
                     lr, beta1, beta2, eps, weight_decay, step, ptr(grad_scale_tensor), grad_scale, int(zero_grad),
                     stream_ptr())
        return
    # library-kernel path (CPU plumbing and the baseline arm): processed in slices so
    # that the temporaries stay small next to the optimizer state
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    chunk = 1 << 26
    for lo in range(0, n, chunk):
        sl = slice(lo, min(n, lo + chunk))
        g = grad[sl] * grad_scale
        if grad_scale_tensor is not None:
            g = g * grad_scale_tensor
        m[sl].mul_(beta1).add_(g, alpha=1 - beta1)
        v[sl].mul_(beta2).addcmul_(g, g, value=1 - beta2)
        denom = (v[sl] / bc2).sqrt_().add_(eps)
        master[sl].mul_(1 - lr * weight_decay).addcdiv_(m[sl], denom, value=-lr / bc1)
        if zero_grad:
            grad[sl].zero_()
        if param_bf16 is not None:
            param_bf16[sl].copy_(master[sl])


def sumsq_(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[0] += sum(x**2) for a flat fp32 tensor."""
    if x.numel() == 0:
        return
    if use_native(x):
        _native.call("dd_sumsq_f32", x.data_ptr(), x.numel(), out.data_ptr(), stream_ptr())
    else:
        for lo in range(0, x.numel(), 1 << 26):
            c = x[lo:lo + (1 << 26)]
            out += (c.float() * c.float()).sum()


def accumulate_f32_(acc: torch.Tensor, g: torch.Tensor, scale: float = 1.0) -> None:
    """``acc += scale * g`` with a flat fp32 accumulator and a gradient of any
    float dtype (one fused cast-and-add kernel for contiguous bf16 on a GPU)."""
    if use_native(g) and g.dtype == torch.bfloat16 and g.is_contiguous() and acc.is_contiguous():
        _native.call("dd_cast_bf16_f32", g.data_ptr(), acc.data_ptr(), g.numel(), float(scale), 1, stream_ptr())
    else:
        acc.add_(g.reshape(-1).to(acc.dtype), alpha=scale)
