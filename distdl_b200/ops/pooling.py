"""Local average / max pooling of ``[batch, channel, *space]`` tensors on this library's kernels
(``csrc/pooling.cu``): the input may be a strided view, so the crop that follows the halo
exchange costs no copy.  Stands where the reference calls ``torch.nn.functional.*_pool*d``
(``src/distdl/nn/pooling.py:150-170``)."""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ._util import stream_ptr

_i3 = ctypes.c_int * 3
_l3 = ctypes.c_longlong * 3
_v, _ll, _i = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
_native.declare("dd_pool_fwd", [_v, _v, _v, _ll, _i3, _i3, _i3, _i3, _i3, _ll, _l3, _i, _i, _v])
_native.declare("dd_pool_bwd", [_v, _v, _v, _ll, _i3, _i3, _i3, _i3, _i3, _i, _i, _v])
_DT = {torch.bfloat16: 0, torch.float32: 1}


def usable(x: torch.Tensor) -> bool:
    """CUDA tensor of a supported type whose batch and channel dimensions collapse into one
    (true for every view that only slices the spatial dimensions)."""
    if not x.is_cuda or x.dtype not in _DT or x.dim() < 3 or x.dim() > 5 or x.numel() == 0:
        return False
    return x.shape[0] == 1 or x.stride(0) == x.shape[1] * x.stride(1)


def _three(v, fill):
    v = [int(a) for a in v]
    return [fill] * (3 - len(v)) + v


class _PoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kind, kernel, stride, dilation):
        nd = x.dim() - 2
        planes = x.shape[0] * x.shape[1]
        n_in = _three(x.shape[2:], 1)
        k, s, d = _three(kernel, 1), _three(stride, 1), _three(dilation, 1)
        n_out = [(n_in[i] - (k[i] - 1) * d[i] - 1) // s[i] + 1 for i in range(3)]
        if min(n_out) <= 0:
            raise ValueError("pooling window larger than the input")
        xs = _three(x.stride()[2:], 0)
        y = torch.empty(tuple(x.shape[:2]) + tuple(n_out[3 - nd:]), dtype=x.dtype, device=x.device)
        is_max = int(kind == "max")
        arg = torch.empty(y.shape, dtype=torch.int32, device=x.device) if is_max else None
        _native.call("dd_pool_fwd", x.data_ptr(), y.data_ptr(), arg.data_ptr() if is_max else None, planes, _i3(*n_in),
                     _i3(*n_out), _i3(*k), _i3(*s), _i3(*d), x.stride(1), _l3(*xs), is_max, _DT[x.dtype], stream_ptr())
        ctx.geom = (planes, n_in, n_out, k, s, d, is_max, tuple(x.shape))
        if is_max:
            ctx.save_for_backward(arg)
        return y

    @staticmethod
    def backward(ctx, dy):
        planes, n_in, n_out, k, s, d, is_max, shape = ctx.geom
        arg = ctx.saved_tensors[0] if is_max else None
        dy = dy.contiguous()
        dx = torch.empty(shape, dtype=dy.dtype, device=dy.device)
        _native.call("dd_pool_bwd", dy.data_ptr(), arg.data_ptr() if is_max else None, dx.data_ptr(), planes,
                     _i3(*n_in), _i3(*n_out), _i3(*k), _i3(*s), _i3(*d), is_max, _DT[dy.dtype], stream_ptr())
        return dx, None, None, None, None


def pool(x: torch.Tensor, kind: str, kernel, stride, dilation=None) -> torch.Tensor:
    """``kind`` = ``"avg"`` (divides by the window volume) or ``"max"``; no padding, floor mode."""
    nd = x.dim() - 2
    dilation = [1] * nd if dilation is None else dilation
    return _PoolFn.apply(x, kind, tuple(kernel), tuple(stride), tuple(dilation))
