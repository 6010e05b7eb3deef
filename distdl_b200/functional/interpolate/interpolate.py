"""Autograd wrapper of the native interpolation kernels
(``src/distdl/functional/interpolate/interpolate.py:18-145`` in the reference,
whose kernels are CPU-only; here CPU and CUDA tensors are both served by
``csrc/interpolate.cu``)."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from ... import _native

_v, _i, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
_IP, _DP = ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_double)
_native.declare("dd_interpolate", [_i, _i, _i, _i, _i, _v, _v, _ll, _IP, _IP, _IP, _IP, _IP, _IP, _DP, _i, _v])

_MODES = {"nearest": 0, "constant": 0, "linear": 1, "bilinear": 1, "trilinear": 1}


def _ints(a):
    a = [int(v) for v in a]
    return (ctypes.c_int * len(a))(*a)


def _call(x, y, adjoint, mode, x_off, y_off, in_global, out_global, scale, align_corners):
    nd = x.dim() - 2
    BC = x.shape[0] * x.shape[1]
    cuda = int(x.is_cuda)
    dtype = {torch.float32: 0, torch.float64: 1}[x.dtype]
    stream = torch.cuda.current_stream().cuda_stream if cuda else 0
    sc = (ctypes.c_double * nd)(*[float(s) for s in scale])
    _native.launch_count += cuda
    _native.check(_native.lib().dd_interpolate(
        cuda, _MODES[mode], int(adjoint), dtype, nd, x.data_ptr(), y.data_ptr(), BC, _ints(x.shape[2:]),
        _ints(y.shape[2:]), _ints(x_off), _ints(y_off), _ints(in_global), _ints(out_global), sc,
        int(bool(align_corners)), stream), "dd_interpolate")


def _steps(in_global, out_global, scale_factor, align_corners):
    """Source step per output index, per dimension."""
    out = []
    for d, (n_in, n_out) in enumerate(zip(in_global, out_global)):
        sf = None if scale_factor is None else (scale_factor[d] if np.ndim(scale_factor) else scale_factor)
        out.append(1.0 / float(sf) if (sf is not None and sf > 0 and not align_corners) else float(n_in) / float(n_out))
    return out


class InterpolateFunction(torch.autograd.Function):
    """``y_local = I(x_local)`` where both are slabs of global tensors.

    ``x_local`` [batch, channel, *in_local] starts at global spatial index
    ``x_local_start``; the result covers ``[y_local_start, y_local_stop)`` of the
    global output of spatial shape ``y_global_shape``.  Shapes are spatial only
    or full (the last ``x.dim() - 2`` entries are used)."""

    @staticmethod
    def forward(ctx, x, x_local_start, x_local_stop, x_global_shape, y_local_start, y_local_stop, y_global_shape,
                scale_factor, mode, align_corners):
        nd = x.dim() - 2
        tail = lambda a: [int(v) for v in list(a)[-nd:]]  # noqa: E731
        x_off, y_off = tail(x_local_start), tail(y_local_start)
        in_g, out_g = tail(x_global_shape), tail(y_global_shape)
        out_local = [b - a for a, b in zip(y_off, tail(y_local_stop))]
        xc = x.contiguous()
        if xc.dtype not in (torch.float32, torch.float64):
            xc = xc.float()
        y = torch.empty(list(x.shape[:2]) + out_local, dtype=xc.dtype, device=x.device)
        steps = _steps(in_g, out_g, scale_factor, align_corners)
        _call(xc, y, False, mode, x_off, y_off, in_g, out_g, steps, align_corners)
        ctx.cfg = (mode, x_off, y_off, in_g, out_g, steps, align_corners, tuple(xc.shape), x.dtype)
        return y.to(x.dtype)

    @staticmethod
    def backward(ctx, gy):
        mode, x_off, y_off, in_g, out_g, steps, align_corners, xshape, xdtype = ctx.cfg
        g = gy.contiguous()
        if g.dtype not in (torch.float32, torch.float64):
            g = g.float()
        gx = torch.zeros(xshape, dtype=g.dtype, device=g.device)
        _call(gx, g, True, mode, x_off, y_off, in_g, out_g, steps, align_corners)
        return (gx.to(xdtype),) + (None,) * 9


def interpolate(x, x_local_start, x_local_stop, x_global_shape, y_local_start, y_local_stop, y_global_shape,
                scale_factor=None, mode="linear", align_corners=False):
    return InterpolateFunction.apply(x, x_local_start, x_local_stop, x_global_shape, y_local_start, y_local_stop,
                                     y_global_shape, scale_factor, mode, align_corners)
