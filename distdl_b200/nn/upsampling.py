"""Upsampling of spatially partitioned tensors (``src/distdl/nn/upsampling.py:16-258``)."""
import numpy as np
import torch.nn.functional as F

from ..utilities.slicing import compute_start_index, compute_stop_index
from ..utilities.torch import TensorStructure, distdl_padding_to_torch_padding
from .halo_exchange import HaloExchange
from .interpolate import Interpolate
from .mixins.interpolate_mixin import InterpolateMixin
from .module import Module


class DistributedUpsample(Module, InterpolateMixin):
    r"""``torch.nn.Upsample`` for ``[batch, channel, *space]`` tensors whose spatial
    dimensions are split over ``P_x``.  Give ``size`` (global output spatial shape)
    or ``scale_factor``; ``mode`` in ``nearest`` / ``linear`` (cubic is not
    implemented).  Each worker produces its balanced slab of the output: it
    fetches, through a halo exchange, the input rows of its neighbours that its
    output rows sample, then interpolates locally in global coordinates."""

    def __init__(self, P_x, buffer_manager=None, size=None, scale_factor=None, mode="linear", align_corners=False):
        super().__init__()
        if mode == "cubic":
            raise NotImplementedError("Cubic interpolation is not implemented.")
        if mode not in ("nearest", "linear"):
            raise NotImplementedError(f"Mode {mode!r} is not supported.")
        if (size is None) == (scale_factor is None):
            raise ValueError("Exactly one of size and scale_factor must be given.")
        self.P_x, self.size, self.scale_factor = P_x, size, scale_factor
        self.mode, self.align_corners = mode, align_corners
        self.buffer_manager = buffer_manager or self._distdl_backend.BufferManager()
        self.interp_layer = None
        self.halo_layer = None

    def _needed(self, index, x_global, y_global, sf):
        shape = self.P_x.shape
        y_lo, y_hi = compute_start_index(shape, index, y_global), compute_stop_index(shape, index, y_global)
        x_lo, x_hi = compute_start_index(shape, index, x_global), compute_stop_index(shape, index, x_global)
        lo, hi = self._compute_needed_range(y_lo, y_hi, x_global, y_global, sf, self.mode, self.align_corners)
        empty = y_hi <= y_lo
        left = np.where(empty, 0, np.maximum(0, x_lo - lo))
        right = np.where(empty, 0, np.maximum(0, hi - x_hi))
        return np.stack([left, right], axis=1).astype(int), x_lo, x_hi, y_lo, y_hi

    def _distdl_module_setup(self, input):
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])
        if not self.P_x.active:
            return
        be = self._distdl_backend
        g = be.assemble_global_tensor_structure(TensorStructure(input[0]), self.P_x)
        x_global = np.asarray(g.shape, dtype=int)
        dims = len(x_global)
        nd = dims - 2
        if self.size is not None:
            size = np.atleast_1d(np.asarray(self.size, dtype=int))
            size = size if size.size == nd else np.repeat(size, nd)
            y_global = np.concatenate([x_global[:2], size])
            sf = [None] * dims
        else:
            s = np.atleast_1d(np.asarray(self.scale_factor, dtype=float))
            s = s if s.size == nd else np.repeat(s, nd)
            y_global = np.concatenate([x_global[:2], np.floor(x_global[2:] * s).astype(int)])
            sf = [None, None] + [float(v) for v in s]
        idx = [int(i) for i in self.P_x.index]
        halo, x_lo, x_hi, y_lo, y_hi = self._needed(idx, x_global, y_global, sf)
        send = np.zeros_like(halo)
        for d in range(dims):
            for side, step in ((0, -1), (1, 1)):
                j = list(idx)
                j[d] += step
                if 0 <= j[d] < int(self.P_x.shape[d]):
                    send[d, side] = self._needed(j, x_global, y_global, sf)[0][d, 1 - side]
        self.pad_tuple = distdl_padding_to_torch_padding(halo)
        self.halo_layer = HaloExchange(self.P_x, halo, halo, send, self.buffer_manager)
        self.interp_layer = Interpolate(x_lo - halo[:, 0], x_hi + halo[:, 1], x_global, y_lo, y_hi, y_global,
                                        scale_factor=None if self.scale_factor is None else sf[2:], mode=self.mode,
                                        align_corners=self.align_corners)

    def _distdl_module_teardown(self, input):
        self.halo_layer = self.interp_layer = None
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if not self.P_x.active:
            return input
        x = F.pad(input, self.pad_tuple, mode="constant", value=0)
        x = self.halo_layer(x)
        return self.interp_layer(x)
