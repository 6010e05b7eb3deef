"""LayerNorm / RMSNorm over a feature dimension that is split across workers,
with the statistics exchange inside the norm kernel.

Each member normalises its local features ``x [rows, d_local]`` with the
statistics of the full rows: one kernel writes per-row partial sums to the
symmetric staging buffer, passes a per-CTA team barrier, reads the partials of
all members over NVLink and normalises.  The backward kernel exchanges the two
per-row sums of the input gradient the same way.  Replaces the two
``AllSumReduce`` calls around the local arithmetic of the reference
(``src/distdl/nn/layernorm.py:218-247``) and is exact for unequal shards.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from . import collectives, symm

c_void_p, c_int, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_IP = ctypes.POINTER(c_int)
_native.declare("dd_split_norm_fwd", symm._TEAM + [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                   c_int, c_float, _IP, c_void_p])
_native.declare("dd_split_norm_bwd", symm._TEAM + [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                   c_void_p, c_int, c_int, c_float, _IP, c_void_p])


def usable(x: torch.Tensor, w, b, ranks) -> bool:
    d = x.shape[-1]
    rows = x.numel() // max(d, 1)
    return (x.is_cuda and x.dtype == torch.bfloat16 and d % 8 == 0 and rows > 0 and 1 < len(ranks) <= 8
            and collectives.available(ranks) and symm.heap_ready() and rows * 16 <= symm.heap().staging_bytes
            and (w is None or (w.dtype == torch.bfloat16 and w.numel() == d))
            and (b is None or (b.dtype == torch.bfloat16 and b.numel() == d)))


def _ptr(t):
    return 0 if t is None else t.data_ptr()


class _SplitNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps, rms, ranks, n_global):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        wc = None if w is None else w.reshape(-1).contiguous()
        bc = None if b is None else b.reshape(-1).contiguous()
        y = torch.empty_like(x2)
        stats = torch.empty(rows, 2, dtype=torch.float32, device=x.device)
        collectives._launch("dd_split_norm_fwd", symm.heap(), list(ranks), int(rms), x2.data_ptr(), _ptr(wc), _ptr(bc),
                            y.data_ptr(), stats.data_ptr(), rows, d, float(eps))
        ctx.save_for_backward(x2, wc, stats)
        ctx.rms, ctx.ranks, ctx.n_global = rms, tuple(ranks), float(n_global)
        ctx.wshape = None if w is None else w.shape
        ctx.bshape = None if b is None else b.shape
        ctx.xshape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, wc, stats = ctx.saved_tensors
        rows, d = x2.shape
        dy2 = dy.reshape(rows, d)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        want_w = ctx.wshape is not None and ctx.needs_input_grad[1]
        want_b = ctx.bshape is not None and ctx.needs_input_grad[2]
        dw = torch.zeros(d, dtype=torch.float32, device=x2.device) if want_w else None
        db = torch.zeros(d, dtype=torch.float32, device=x2.device) if want_b else None
        collectives._launch("dd_split_norm_bwd", symm.heap(), list(ctx.ranks), int(ctx.rms), dy2.data_ptr(),
                            x2.data_ptr(), _ptr(wc), stats.data_ptr(), dx.data_ptr(), _ptr(dw), _ptr(db), rows, d,
                            ctx.n_global)
        gw = dw.to(x2.dtype).view(ctx.wshape) if want_w else None
        gb = db.to(x2.dtype).view(ctx.bshape) if want_b else None
        return dx.view(ctx.xshape), gw, gb, None, None, None, None


def split_norm(x, w, b, eps, ranks, n_global, rms=False):
    """Norm of ``x [..., d_local]`` over the full feature dimension of ``n_global``
    elements that the workers ``ranks`` (world ranks, the caller among them) hold
    in pieces; ``w`` / ``b`` are the local pieces of the affine parameters."""
    return _SplitNormFn.apply(x, w, b, eps, rms, tuple(ranks), n_global)
