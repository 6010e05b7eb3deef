"""Fused softmax-cross-entropy: one kernel computes the per-row loss and
overwrites the logits with their gradient, so the backward pass of the loss is
free and the fp32 probabilities are never materialised."""
from __future__ import annotations

import torch

from .. import _native
from ._util import stream_ptr, use_native


class _XentFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, vocab, scale, unit_grad):
        # logits [rows, ld] bf16, contiguous; destroyed (replaced by d loss / d logits * scale)
        rows, ld = logits.shape
        if targets.dtype != torch.int64:
            raise TypeError(f"cross_entropy_: targets must be int64 (the kernel reads 8-byte ids), got {targets.dtype}")
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        _native.call("dd_xent", logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), rows, vocab, ld,
                     float(scale), stream_ptr())
        # the kernel wrote through a raw pointer: tell autograd that the storage changed, so that any
        # other function that saved these logits for its backward fails loudly instead of reading gradients
        torch.autograd.graph.increment_version(logits)
        ctx.save_for_backward(logits)
        ctx.unit_grad = unit_grad
        return loss.sum() * scale

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        if ctx.unit_grad:  # caller promises d(total)/d(loss) == 1: no host sync, no extra pass
            return dlogits, None, None, None, None
        return dlogits * g.to(dlogits.dtype), None, None, None, None


def cross_entropy_(logits: torch.Tensor, targets: torch.Tensor, vocab: int = None, scale: float = None,
                   unit_grad: bool = False):
    """Mean (or ``scale``-weighted sum) token cross-entropy.

    ``logits`` [rows, ld] (columns >= ``vocab`` are padding) is consumed: on
    CUDA its storage is overwritten with the gradient.  ``scale`` defaults to
    ``1 / rows``.  ``unit_grad=True`` promises that the returned loss is
    back-propagated with gradient 1 (fold any loss scaling into ``scale``),
    which lets backward hand the stored gradient through untouched.
    """
    rows, ld = logits.shape
    vocab = vocab or ld
    if scale is None:
        scale = 1.0 / rows
    if use_native(logits) and logits.dtype == torch.bfloat16 and ld % 8 == 0 and logits.is_contiguous():
        return _XentFn.apply(logits, targets.contiguous(), vocab, scale, unit_grad)
    return torch.nn.functional.cross_entropy(logits[:, :vocab].float(), targets, reduction="sum",
                                             ignore_index=-100) * scale
