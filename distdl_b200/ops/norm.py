"""Fused RMSNorm / LayerNorm (forward + backward) kernels.

Replaces ``torch.nn.functional.layer_norm`` and the optional
``flash_attn.ops`` fused norms of the reference
(``src/distdl/nn/layernorm.py:311-319``, ``src/distdl/nn/layernorm_zero.py:298-301``,
``src/distdl/nn/rmsnorm_zero.py:333-347``).  Statistics are kept in fp32.
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, stream_ptr, use_native

_scratch = {}


def _partial_buffer(rows: int, d: int, device) -> torch.Tensor:
    """Scratch for the per-CTA dw/db partial sums, cached per device and grown on demand."""
    parts = _native.lib().dd_norm_bwd_parts(rows)
    need = parts * 2 * d
    buf = _scratch.get(device)
    if buf is None or buf.numel() < need:
        buf = torch.empty(need, dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps, rms):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        stats = torch.empty(rows, 2, dtype=torch.float32, device=x.device)
        _native.call("dd_norm_fwd", int(rms), x2.data_ptr(), 0, 0, ptr(w), ptr(b), y.data_ptr(), stats.data_ptr(),
                     rows, d, float(eps), stream_ptr())
        ctx.save_for_backward(x2, w, stats)
        ctx.rms = rms
        ctx.wref, ctx.bref = w, b
        ctx.xshape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, stats = ctx.saved_tensors
        d = x2.shape[-1]
        rows = x2.shape[0]
        dy2 = dy.reshape(-1, d)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        want_w = w is not None and ctx.needs_input_grad[1]
        want_b = ctx.bref is not None and ctx.needs_input_grad[2]
        dw = db = None
        dw_buf = db_buf = None
        acc = 0
        partial = None
        if want_w or want_b:
            partial = _partial_buffer(rows, d, x2.device)
            mgw = getattr(ctx.wref, "main_grad", None) if want_w else None
            mgb = getattr(ctx.bref, "main_grad", None) if want_b else None
            if mgw is not None or mgb is not None:
                acc = 1
                dw_buf, db_buf = mgw, mgb
                if want_w and mgw is None:
                    raise RuntimeError("main_grad must be set on both weight and bias or on neither")
            else:
                if want_w:
                    dw_buf = torch.empty(d, dtype=torch.float32, device=x2.device)
                if want_b:
                    db_buf = torch.empty(d, dtype=torch.float32, device=x2.device)
        _native.call("dd_norm_bwd", int(ctx.rms), dy2.data_ptr(), x2.data_ptr(), ptr(w), stats.data_ptr(), 0,
                     dx.data_ptr(), ptr(dw_buf), ptr(db_buf), ptr(partial), acc, rows, d, stream_ptr())
        if not acc:
            if want_w:
                dw = dw_buf.to(w.dtype).view(w.shape)
            if want_b:
                db = db_buf.to(ctx.bref.dtype).view(ctx.bref.shape)
        return dx.view(ctx.xshape), dw, db, None, None


class _AddNormFn(torch.autograd.Function):
    """``s = x + res; y = norm(s)`` in one kernel, returning both: the residual add of a transformer
    block rides along with the norm that follows it (forward: one pass instead of two; backward: the
    gradient of ``s`` that arrives from the residual stream is added inside the norm's backward
    kernel)."""

    @staticmethod
    def forward(ctx, x, res, w, b, eps, rms):
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        r2 = res.reshape(-1, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if not r2.is_contiguous():
            r2 = r2.contiguous()
        rows = x2.shape[0]
        xsum = torch.empty_like(x2)
        y = torch.empty_like(x2)
        stats = torch.empty(rows, 2, dtype=torch.float32, device=x.device)
        _native.call("dd_norm_fwd", int(rms), x2.data_ptr(), r2.data_ptr(), xsum.data_ptr(), ptr(w), ptr(b),
                     y.data_ptr(), stats.data_ptr(), rows, d, float(eps), stream_ptr())
        ctx.save_for_backward(xsum, w, stats)
        ctx.rms = rms
        ctx.wref, ctx.bref = w, b
        ctx.xshape = x.shape
        ctx.set_materialize_grads(False)
        return xsum.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, dsum, dy):
        xs, w, stats = ctx.saved_tensors
        if dy is None:
            return dsum, dsum, None, None, None, None
        d = xs.shape[-1]
        rows = xs.shape[0]
        dy2 = dy.reshape(-1, d)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if dsum is not None:
            dres = dsum.reshape(-1, d)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        dx = torch.empty_like(xs)
        want_w = w is not None and ctx.needs_input_grad[2]
        want_b = ctx.bref is not None and ctx.needs_input_grad[3]
        dw = db = dw_buf = db_buf = partial = None
        acc = 0
        if want_w or want_b:
            partial = _partial_buffer(rows, d, xs.device)
            mgw = getattr(ctx.wref, "main_grad", None) if want_w else None
            mgb = getattr(ctx.bref, "main_grad", None) if want_b else None
            if mgw is not None or mgb is not None:
                acc = 1
                dw_buf, db_buf = mgw, mgb
                if want_w and mgw is None:
                    raise RuntimeError("main_grad must be set on both weight and bias or on neither")
            else:
                if want_w:
                    dw_buf = torch.empty(d, dtype=torch.float32, device=xs.device)
                if want_b:
                    db_buf = torch.empty(d, dtype=torch.float32, device=xs.device)
        _native.call("dd_norm_bwd", int(ctx.rms), dy2.data_ptr(), xs.data_ptr(), ptr(w), stats.data_ptr(), ptr(dres),
                     dx.data_ptr(), ptr(dw_buf), ptr(db_buf), ptr(partial), acc, rows, d, stream_ptr())
        if not acc:
            if want_w:
                dw = dw_buf.to(w.dtype).view(w.shape)
            if want_b:
                db = db_buf.to(ctx.bref.dtype).view(ctx.bref.shape)
        dx = dx.view(ctx.xshape)
        return dx, dx, dw, db, None, None


def _ok(x, w, b):
    d = x.shape[-1]
    return (use_native(x) and x.dtype == torch.bfloat16 and d % 8 == 0 and d <= 8192
            and (w is None or (w.dtype == torch.bfloat16 and w.numel() == d))
            and (b is None or (b.dtype == torch.bfloat16 and b.numel() == d)))


def rms_norm(x, weight=None, eps: float = 1e-6, bias=None):
    """y = x * rsqrt(mean(x^2) + eps) * weight (+ bias) over the last dimension."""
    if _ok(x, weight, bias):
        return _NormFn.apply(x, weight, bias, eps, True)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    """LayerNorm over the last dimension."""
    if _ok(x, weight, bias):
        return _NormFn.apply(x, weight, bias, eps, False)
    d = x.shape[-1]
    return torch.nn.functional.layer_norm(x, (d,), None if weight is None else weight.reshape(d),
                                          None if bias is None else bias.reshape(d), eps)


def add_rms_norm(x, res, weight=None, eps: float = 1e-6, bias=None):
    """``(x + res, rms_norm(x + res))``: the residual add fused into the norm that follows it."""
    if _ok(x, weight, bias) and res.dtype == x.dtype and res.shape == x.shape:
        return _AddNormFn.apply(x, res, weight, bias, eps, True)
    s = x + res
    return s, rms_norm(s, weight, eps, bias)


def add_layer_norm(x, res, weight=None, bias=None, eps: float = 1e-5):
    """``(x + res, layer_norm(x + res))``: the residual add fused into the norm that follows it."""
    if _ok(x, weight, bias) and res.dtype == x.dtype and res.shape == x.shape:
        return _AddNormFn.apply(x, res, weight, bias, eps, False)
    s = x + res
    return s, layer_norm(s, weight, bias, eps)
