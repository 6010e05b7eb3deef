"""Sequential interpolation of a sub-tensor in global coordinates
(``src/distdl/nn/interpolate.py:6-80``)."""
import torch

from ..functional.interpolate import interpolate


class Interpolate(torch.nn.Module):
    r"""Interpolates the slab ``[x_local_start, x_local_stop)`` of a global tensor
    of shape ``x_global_shape`` onto the slab ``[y_local_start, y_local_stop)`` of
    the global output ``y_global_shape``; ``mode`` in ``nearest`` / ``linear``."""

    def __init__(self, x_local_start, x_local_stop, x_global_shape, y_local_start, y_local_stop, y_global_shape,
                 scale_factor=None, mode="nearest", align_corners=False):
        super().__init__()
        if mode not in ("nearest", "linear", "constant", "bilinear", "trilinear"):
            raise NotImplementedError(f"interpolation mode {mode!r}")
        self.x_local_start, self.x_local_stop, self.x_global_shape = x_local_start, x_local_stop, x_global_shape
        self.y_local_start, self.y_local_stop, self.y_global_shape = y_local_start, y_local_stop, y_global_shape
        self.scale_factor, self.mode, self.align_corners = scale_factor, mode, align_corners

    def forward(self, input):
        return interpolate(input, self.x_local_start, self.x_local_stop, self.x_global_shape, self.y_local_start,
                           self.y_local_stop, self.y_global_shape, self.scale_factor, self.mode, self.align_corners)
