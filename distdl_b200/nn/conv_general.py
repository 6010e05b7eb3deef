"""Convolution with channels *and* space partitioned
(``src/distdl/nn/conv_general.py:19-523``)."""
import numpy as np
import torch
import torch.nn.functional as F

from ..utilities.slicing import assemble_slices, compute_subshape
from ..utilities.torch import TensorStructure, distdl_padding_to_torch_padding, zero_volume_tensor
from .broadcast import Broadcast
from .conv_channel import _CONV, _expand
from .halo_exchange import HaloExchange
from .mixins.conv_mixin import ConvMixin
from .mixins.halo_mixin import HaloMixin
from .module import Module
from .sum_reduce import SumReduce


class DistributedGeneralConvBase(Module, HaloMixin, ConvMixin):
    r"""``P_x = [1, P_ci, *P_space]``, ``P_y = [1, P_co, *P_space]``,
    ``P_w = [P_co, P_ci, *P_space]``.  Forward: halo exchange of the input on
    ``P_x`` (spatial neighbours), broadcast of the padded input along the
    output-channel dimension of ``P_w``, local convolution on every worker of
    ``P_w`` (the weight block ``[co/P_co, ci/P_ci, *k]`` lives there; bias only
    where the input-channel index is 0), sum-reduction over the input-channel
    dimension onto ``P_y``."""

    num_dimensions = None

    def __init__(self, P_x, P_y, P_w, in_channels, out_channels, kernel_size, stride=1, padding=0,
                 padding_mode="zeros", dilation=1, groups=1, bias=True, buffer_manager=None, device=None, dtype=None):
        super().__init__()
        self.P_x, self.P_y, self.P_w = P_x, P_y, P_w
        self.buffer_manager = buffer_manager or self._distdl_backend.BufferManager()
        if not (P_x.active or P_y.active or P_w.active):
            return
        nd = self.num_dimensions
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride = np.asarray(_expand(kernel_size, nd)), np.asarray(_expand(stride, nd))
        self.padding, self.dilation = np.asarray(_expand(padding, nd)), np.asarray(_expand(dilation, nd))
        self.groups, self.use_bias = groups, bias
        if padding_mode != "zeros":
            raise NotImplementedError("only zero padding is supported")
        device = device if device is not None else (P_w.device if P_w.active else P_x.device)
        # Weights live once per (out-channel, in-channel) block, on the workers of
        # P_w with spatial index 0 (P_wr), and are broadcast to the spatial replicas.
        self.has_bias_here = False
        if P_w.active:
            from ._linear_common import derived_partition
            dim = P_w.dim
            idx = [slice(0, int(P_w.shape[0])), slice(0, int(P_w.shape[1]))] + [slice(0, 1)] * (dim - 2)
            shape = [int(P_w.shape[0]), int(P_w.shape[1])] + [1] * (dim - 2)
            self.P_wr = derived_partition(P_w, idx, shape)
            self.w_broadcast = Broadcast(self.P_wr, P_w, preserve_batch=False)
            self.b_broadcast = Broadcast(self.P_wr, P_w, preserve_batch=False) if bias else None
            co = int(compute_subshape(P_w.shape[0], P_w.index[0], [out_channels])[0])
            ci = int(compute_subshape(P_w.shape[1], P_w.index[1], [in_channels])[0])
            fan_in = in_channels // groups * int(np.prod(self.kernel_size))
            bound = 1.0 / np.sqrt(fan_in)
            self.has_bias_here = bias and int(P_w.index[1]) == 0
            if self.P_wr.active:
                self.weight = torch.nn.Parameter(
                    torch.empty(co, ci // groups, *[int(k) for k in self.kernel_size], device=device,
                                dtype=dtype).uniform_(-bound, bound))
                if self.has_bias_here:
                    self.bias = torch.nn.Parameter(torch.empty(co, device=device, dtype=dtype).uniform_(-bound, bound))
                elif bias:
                    self.register_buffer("bias", zero_volume_tensor(device=device, dtype=dtype, requires_grad=True))
                else:
                    self.register_parameter("bias", None)
            else:
                self.register_buffer("weight", zero_volume_tensor(device=device, dtype=dtype, requires_grad=True))
                if bias:
                    self.register_buffer("bias", zero_volume_tensor(device=device, dtype=dtype, requires_grad=True))
                else:
                    self.register_parameter("bias", None)
        else:
            self.register_buffer("weight", zero_volume_tensor(device=device, dtype=dtype))
            self.register_parameter("bias", None)
        y_view = [int(P_y.shape[1]), 1] + [int(v) for v in P_y.shape[2:]]
        self.P_y_view = P_y.create_cartesian_topology_partition(y_view)
        self.x_broadcast = Broadcast(P_x, P_w, preserve_batch=True)
        self.y_sum_reduce = SumReduce(P_w, self.P_y_view, preserve_batch=True)
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
        if not (self.P_x.active or self.P_y.active or self.P_w.active):
            return input
        x = input
        if self.P_x.active:
            x = F.pad(x, self.pad_tuple, mode="constant", value=0)
            x = self.halo_layer(x)
            x = x[self.needed_slices]
        x = self.x_broadcast(x)
        if self.P_w.active:
            w = self.w_broadcast(self.weight)
            b = self.b_broadcast(self.bias) if self.use_bias else None
            if not self.has_bias_here:
                b = None
            x = _CONV[self.num_dimensions](x, w, b, stride=tuple(int(s) for s in self.stride),
                                           padding=0, dilation=tuple(int(d) for d in self.dilation),
                                           groups=self.groups)
        return self.y_sum_reduce(x)


class DistributedGeneralConv1d(DistributedGeneralConvBase):
    num_dimensions = 1


class DistributedGeneralConv2d(DistributedGeneralConvBase):
    num_dimensions = 2


class DistributedGeneralConv3d(DistributedGeneralConvBase):
    num_dimensions = 3
