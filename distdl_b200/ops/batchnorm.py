"""Local arithmetic of the distributed batch norm: per-feature reductions and the per-feature
affine map of ``[batch, feature, rest...]`` tensors (kernels in ``csrc/batchnorm.cu``), as autograd
functions.  The layer (:mod:`distdl_b200.nn.batchnorm`) moves the per-feature sums between workers
with the SumReduce / Broadcast primitives; these stand where the reference uses ``tensor.sum`` and
element-wise PyTorch operations around those primitives (``src/distdl/nn/batchnorm.py:306-360``)."""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import ptr, stream_ptr, use_native

_v, _i, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_native.declare("dd_bn_reduce", [_v, _v, _v, _i, _i, _ll, _i, _i, _v, _v, _v])
_native.declare("dd_bn_affine", [_v, _v, _v, _v, _v, _v, _i, _i, _ll, _i, _v, _v])
_DT = {torch.bfloat16: 0, torch.float32: 1}


def usable(x: torch.Tensor) -> bool:
    return use_native(x) and x.dtype in _DT and x.dim() >= 2 and x.is_contiguous() and x.numel() > 0


def _geometry(x):
    B, F = int(x.shape[0]), int(x.shape[1])
    R = x.numel() // (B * F)
    return B, F, R


def _stat_shape(x):
    return (1, x.shape[1]) + (1,) * (x.dim() - 2)


def _reduce(x, dy, shift, mode):
    B, F, R = _geometry(x)
    out = torch.zeros(2, F, dtype=torch.float32, device=x.device)
    sh = None if shift is None else shift.reshape(-1).float().contiguous()
    _native.call("dd_bn_reduce", x.data_ptr(), ptr(dy), ptr(sh), B, F, R, mode, _DT[x.dtype], out[0].data_ptr(),
                 out[1].data_ptr(), stream_ptr())
    return out[0], out[1]


def _affine(x, a, m=None, c=None, z=None, e=None):
    B, F, R = _geometry(x)
    y = torch.empty_like(x)
    f = [None if t is None else t.reshape(-1).float().contiguous() for t in (a, m, c, e)]
    _native.call("dd_bn_affine", x.data_ptr(), ptr(z), ptr(f[0]), ptr(f[1]), ptr(f[2]), ptr(f[3]), B, F, R,
                 _DT[x.dtype], y.data_ptr(), stream_ptr())
    return y


class _ChannelSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.xshape = x.shape
        s, _ = _reduce(x, None, None, 0)
        return s.reshape(_stat_shape(x)).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        return g.expand(ctx.xshape)


class _ChannelSqDev(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mean):
        s1, s2 = _reduce(x, None, mean, 1)
        ctx.save_for_backward(x, mean, s1)
        return s2.reshape(_stat_shape(x)).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        x, mean, s1 = ctx.saved_tensors
        gf = g.reshape(-1).float()
        dx = _affine(x, 2.0 * gf, m=mean) if ctx.needs_input_grad[0] else None
        dmean = (-2.0 * gf * s1).reshape(mean.shape).to(mean.dtype) if ctx.needs_input_grad[1] else None
        return dx, dmean


class _Normalize(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mean, var, gamma, beta, eps):
        rstd = torch.rsqrt(var.reshape(-1).float() + eps)
        g = torch.ones_like(rstd) if gamma is None else gamma.reshape(-1).float()
        ctx.save_for_backward(x, mean, rstd, g)
        ctx.meta = (gamma is not None, beta is not None, mean.shape, mean.dtype,
                    None if gamma is None else (gamma.shape, gamma.dtype),
                    None if beta is None else (beta.shape, beta.dtype))
        return _affine(x, g * rstd, m=mean, c=beta)

    @staticmethod
    def backward(ctx, dy):
        x, mean, rstd, g = ctx.saved_tensors
        has_g, has_b, mshape, mdtype, gmeta, bmeta = ctx.meta
        dy = dy.contiguous()
        sdy, sdyx = _reduce(x, dy, mean, 2)
        dx = _affine(dy, g * rstd) if ctx.needs_input_grad[0] else None
        dmean = (-g * rstd * sdy).reshape(mshape).to(mdtype) if ctx.needs_input_grad[1] else None
        dvar = (-0.5 * g * rstd.pow(3) * sdyx).reshape(mshape).to(mdtype) if ctx.needs_input_grad[2] else None
        dgamma = (rstd * sdyx).reshape(gmeta[0]).to(gmeta[1]) if has_g and ctx.needs_input_grad[3] else None
        dbeta = sdy.reshape(bmeta[0]).to(bmeta[1]) if has_b and ctx.needs_input_grad[4] else None
        return dx, dmean, dvar, dgamma, dbeta, None


def channel_sum(x):
    """Sum over every dimension but the feature dimension (1), kept as ``[1, F, 1, ...]``."""
    if usable(x):
        return _ChannelSum.apply(x)
    return x.sum([d for d in range(x.dim()) if d != 1], keepdim=True)


def channel_sqdev(x, mean):
    """``sum((x - mean) ** 2)`` over every dimension but the feature dimension; ``mean`` is ``[1, F, 1, ...]``."""
    if usable(x) and mean.numel() == x.shape[1]:
        return _ChannelSqDev.apply(x, mean)
    return ((x - mean) ** 2).sum([d for d in range(x.dim()) if d != 1], keepdim=True)


def normalize(x, mean, var, gamma=None, beta=None, eps: float = 1e-5):
    """``gamma * (x - mean) / sqrt(var + eps) + beta`` with per-feature ``[1, F, 1, ...]`` statistics."""
    if usable(x) and mean.numel() == x.shape[1] and var.numel() == x.shape[1] \
            and (gamma is None or gamma.numel() == x.shape[1]) and (beta is None or beta.numel() == x.shape[1]):
        return _Normalize.apply(x, mean, var, gamma, beta, eps)
    y = (x - mean) / torch.sqrt(var + eps)
    if gamma is not None:
        y = gamma * y
    if beta is not None:
        y = y + beta
    return y
