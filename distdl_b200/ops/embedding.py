"""Embedding gather / scatter-add kernels (replace ``F.embedding`` of
``src/distdl/nn/embedding.py:244`` and ``src/distdl/nn/embedding_zero.py:271``)."""
from __future__ import annotations

import torch

from .. import _native
from ._util import stream_ptr, use_native


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1).contiguous()
        d = table.shape[-1]
        out = torch.empty(flat.numel(), d, dtype=table.dtype, device=table.device)
        _native.call("dd_embedding_fwd", flat.data_ptr(), table.data_ptr(), out.data_ptr(), flat.numel(), d,
                     table.shape[0], stream_ptr())
        ctx.save_for_backward(flat)
        ctx.tref = table
        ctx.ishape = ids.shape
        return out.view(*ids.shape, d)

    @staticmethod
    def backward(ctx, dout):
        (flat,) = ctx.saved_tensors
        table = ctx.tref
        d = table.shape[-1]
        d2 = dout.reshape(-1, d).contiguous()
        mg = getattr(table, "main_grad", None)
        if mg is not None:
            _native.call("dd_embedding_bwd", flat.data_ptr(), d2.data_ptr(), mg.data_ptr(), flat.numel(), d,
                         table.shape[0], stream_ptr())
            return None, None
        g = torch.zeros(table.shape, dtype=torch.float32, device=table.device)
        _native.call("dd_embedding_bwd", flat.data_ptr(), d2.data_ptr(), g.data_ptr(), flat.numel(), d,
                     table.shape[0], stream_ptr())
        return None, g.to(table.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor, padding_idx=None) -> torch.Tensor:
    if (use_native(table) and table.dtype == torch.bfloat16 and table.dim() == 2 and table.shape[1] % 8 == 0
            and table.is_contiguous() and ids.dtype == torch.int64 and padding_idx is None):
        return _EmbeddingFn.apply(ids, table)
    return torch.nn.functional.embedding(ids, table, padding_idx=padding_idx)
