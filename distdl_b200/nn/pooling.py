"""Pooling on spatially partitioned tensors (``src/distdl/nn/pooling.py:13-338``)."""
import numpy as np
import torch.nn.functional as F

from ..utilities.slicing import assemble_slices
from ..utilities.torch import TensorStructure, distdl_padding_to_torch_padding
from .conv_feature import _per_dim
from .halo_exchange import HaloExchange
from .mixins.halo_mixin import HaloMixin
from .mixins.pooling_mixin import PoolingMixin
from .module import Module


class DistributedPoolBase(Module, HaloMixin, PoolingMixin):
    r"""Average / max pooling of ``[batch, channel, *space]`` tensors whose spatial
    dimensions are split over ``P_x``: pad at the global boundary (0 for average,
    ``-inf`` for max), exchange halos, crop, and pool locally with ``padding=0``."""

    num_dimensions = None
    pool_kind = None   # "avg" | "max"

    def __init__(self, P_x, kernel_size, stride=1, padding=0, dilation=1, buffer_manager=None, **kwargs):
        super().__init__()
        self.P_x = P_x
        self.buffer_manager = buffer_manager or self._distdl_backend.BufferManager()
        if not P_x.active:
            return
        nd = self.num_dimensions
        exp = lambda v: _per_dim(v, nd)  # noqa: E731
        self.kernel_size, self.stride = exp(kernel_size), exp(stride)
        self.padding, self.dilation = exp(padding), exp(dilation)
        if self.pool_kind == "avg" and np.any(self.dilation != 1):
            raise ValueError("dilation is only supported for max pooling")
        self.pad_value = 0.0 if self.pool_kind == "avg" else float("-inf")
        self.extra = kwargs
        self.halo_layer = None

    def _distdl_module_setup(self, input):
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])
        if not self.P_x.active:
            return
        be = self._distdl_backend
        ts = TensorStructure(input[0])
        g = be.assemble_global_tensor_structure(ts, self.P_x)
        shapes = be.tensor_decomposition.compute_subtensor_shapes_unbalanced(ts, self.P_x)
        halo, recv, send, needed = self._compute_exchange_info(
            g.shape, self.kernel_size, self.stride, self.padding, self.dilation, True, self.P_x.shape,
            self.P_x.index, subtensor_shapes=shapes)
        dims, nd = self.P_x.dim, self.num_dimensions
        gpad = np.concatenate([np.zeros(dims - nd, dtype=int), self.padding])
        local_pad = np.repeat(gpad.reshape(dims, 1), 2, axis=1)
        idx, shape = self.P_x.index, self.P_x.shape
        for d in range(dims):
            if idx[d] != 0:
                local_pad[d, 0] = 0
            if idx[d] != shape[d] - 1:
                local_pad[d, 1] = 0
        self.pad_tuple = distdl_padding_to_torch_padding(local_pad + halo)
        self.halo_layer = HaloExchange(self.P_x, halo + local_pad, recv, send, self.buffer_manager)
        self.needed_slices = assemble_slices(needed[:, 0], needed[:, 1] + local_pad[:, 0] + local_pad[:, 1])

    def _distdl_module_teardown(self, input):
        self.halo_layer = None
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if not self.P_x.active:
            return input
        x = F.pad(input, self.pad_tuple, mode="constant", value=self.pad_value)
        x = self.halo_layer(x)
        x = x[self.needed_slices]
        k = tuple(int(v) for v in self.kernel_size)
        s = tuple(int(v) for v in self.stride)
        if not self.extra and x.is_cuda:
            from ..ops import pooling as pool_ops
            if pool_ops.usable(x):          # this library's kernel reads the cropped view in place
                return pool_ops.pool(x, self.pool_kind, k, s, tuple(int(v) for v in self.dilation))
        if self.pool_kind == "avg":
            fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[self.num_dimensions]
            return fn(x, k, stride=s, padding=0, **self.extra)
        fn = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[self.num_dimensions]
        return fn(x, k, stride=s, padding=0, dilation=tuple(int(v) for v in self.dilation), **self.extra)


class DistributedAvgPool1d(DistributedPoolBase):
    num_dimensions, pool_kind = 1, "avg"


class DistributedAvgPool2d(DistributedPoolBase):
    num_dimensions, pool_kind = 2, "avg"


class DistributedAvgPool3d(DistributedPoolBase):
    num_dimensions, pool_kind = 3, "avg"


class DistributedMaxPool1d(DistributedPoolBase):
    num_dimensions, pool_kind = 1, "max"


class DistributedMaxPool2d(DistributedPoolBase):
    num_dimensions, pool_kind = 2, "max"


class DistributedMaxPool3d(DistributedPoolBase):
    num_dimensions, pool_kind = 3, "max"
