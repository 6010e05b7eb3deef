"""Convolution with the channel dimensions partitioned
(``src/distdl/nn/conv_channel.py:13-338``)."""
import numpy as np
import torch
import torch.nn.functional as F

from ..utilities.slicing import compute_subshape
from .broadcast import Broadcast
from .module import Module
from .sum_reduce import SumReduce


def _expand(v, nd):
    a = np.atleast_1d(np.asarray(v, dtype=int))
    return tuple(int(x) for x in (a if a.size == nd else np.repeat(a, nd)))


_CONV = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}
_CONVT = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}


class DistributedChannelConvBase(Module):
    r"""``P_x = [1, P_ci, 1, ...]`` (input channels split), ``P_y = [1, P_co, 1,
    ...]`` (output channels split), ``P_w = [P_co, P_ci, 1, ...]``.  The input is
    broadcast along the ``P_co`` dimension of the weight grid, every worker
    convolves its channel block (bias only where the input-channel index is 0,
    so it enters the sum once), and the partial outputs are sum-reduced along
    ``P_ci`` onto ``P_y``.  The local convolution is the library kernel."""

    num_dimensions = None

    def __init__(self, P_x, P_y, P_w, in_channels, out_channels, kernel_size, stride=1, padding=0,
                 padding_mode="zeros", dilation=1, groups=1, bias=True, device=None, dtype=None, *args, **kwargs):
        super().__init__()
        self.P_x, self.P_y, self.P_w = P_x, P_y, P_w
        if not (P_x.active or P_y.active or P_w.active):
            return
        nd = self.num_dimensions
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride = _expand(kernel_size, nd), _expand(stride, nd)
        self.padding, self.dilation = _expand(padding, nd), _expand(dilation, nd)
        self.padding_mode, self.groups, self.use_bias = padding_mode, groups, bias
        if P_w.active:
            co = int(compute_subshape(P_w.shape[0], P_w.index[0], [out_channels])[0])
            ci = int(compute_subshape(P_w.shape[1], P_w.index[1], [in_channels])[0])
            has_bias = bias and int(P_w.index[1]) == 0
            cls = {1: torch.nn.Conv1d, 2: torch.nn.Conv2d, 3: torch.nn.Conv3d}[nd]
            self.conv_layer = cls(ci, co, self.kernel_size, stride=self.stride, padding=self.padding,
                                  padding_mode=padding_mode, dilation=self.dilation, groups=groups, bias=has_bias,
                                  device=device if device is not None else P_w.device, dtype=dtype)
            # fan-in of the *global* weight for the initial distribution
            fan_in = in_channels // groups * int(np.prod(self.kernel_size))
            bound = 1.0 / np.sqrt(fan_in)
            with torch.no_grad():
                self.conv_layer.weight.uniform_(-bound, bound)
                if has_bias:
                    self.conv_layer.bias.uniform_(-bound, bound)
        # For the reduction the output partition [1, P_co, 1, ...] is read as the
        # grid [P_co, 1, 1, ...]: it then lines up with P_w = [P_co, P_ci, 1, ...]
        # and the sum runs along the input-channel dimension.
        y_view = [int(P_y.shape[1]), 1] + [int(v) for v in P_y.shape[2:]]
        self.P_y_view = P_y.create_cartesian_topology_partition(y_view)
        self.x_broadcast = Broadcast(P_x, P_w, preserve_batch=True)
        self.y_sum_reduce = SumReduce(P_w, self.P_y_view, preserve_batch=True)

    def forward(self, input):
        if not (self.P_x.active or self.P_y.active or self.P_w.active):
            return input
        x = self.x_broadcast(input)
        if self.P_w.active:
            x = self.conv_layer(x)
        return self.y_sum_reduce(x)


class DistributedChannelConv1d(DistributedChannelConvBase):
    num_dimensions = 1


class DistributedChannelConv2d(DistributedChannelConvBase):
    num_dimensions = 2


class DistributedChannelConv3d(DistributedChannelConvBase):
    num_dimensions = 3
