"""Channel-parallel convolutions in the all-gather form
(``src/distdl/nn/conv_channel_ag.py:64-1129``): the tensor-parallel analogue of
``DistributedLinearAllGather`` for ``[batch, channel, *space]`` tensors."""
import math

import numpy as np
import torch

from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import derived_partition, root_partition
from .all_gather import AllGather
from .broadcast import Broadcast
from .conv_channel import _CONV, _CONVT, _expand
from .module import Module
from .repartition import Repartition


class _ChannelConvNd(Module):
    """Common constructor of the channel all-gather / reduce-scatter convolutions."""

    num_dimensions = None
    transposed = False
    shard = "out"          # which channel dimension of the weight is split over the workers

    def __init__(self, P_x, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1,
                 bias=True, padding_mode="zeros", collect_state=False, output_padding=0, device=None, dtype=None):
        super().__init__()
        if groups <= 0 or in_channels % groups or out_channels % groups:
            raise ValueError("in_channels and out_channels must be divisible by a positive groups")
        if padding_mode != "zeros":
            raise ValueError("only padding_mode='zeros' is supported")
        self.P_x = P_x
        if not P_x.active:
            return
        nd = self.num_dimensions
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride = _expand(kernel_size, nd), _expand(stride, nd)
        self.padding, self.dilation = _expand(padding, nd), _expand(dilation, nd)
        self.output_padding = _expand(output_padding, nd)
        self.groups, self.use_bias, self.collect_state, self.dtype = groups, bias, collect_state, dtype
        device = device if device is not None else P_x.device
        self._device = device
        kw = {"device": device, "dtype": dtype}
        dim, M = P_x.dim, int(P_x.shape[1])
        idx = [slice(0, 1)] * dim
        idx[1] = slice(0, M)
        shape = [1] * dim
        shape[1] = M
        self.P_weight = derived_partition(P_x, idx, shape)
        self.broadcast_weight = Broadcast(self.P_weight, P_x, preserve_batch=False)
        tp = int(P_x.index[1])
        if self.shard == "out":
            out_l = int(compute_subshape(M, tp, [out_channels])[0])
            wshape = ((in_channels, out_l // groups) if self.transposed else (out_l, in_channels // groups))
            bias_len, self.P_bias = out_l, self.P_weight
        else:
            in_l = int(compute_subshape(M, tp, [in_channels])[0])
            wshape = ((in_l, out_channels // groups) if self.transposed else (out_channels, in_l // groups))
            bias_len, self.P_bias = out_channels, root_partition(P_x)
        if self.P_weight.active:
            self.weight = torch.nn.Parameter(torch.empty(*wshape, *self.kernel_size, **kw))
        else:
            self.register_buffer("weight", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
        if bias and self.P_bias.active:
            self.bias = torch.nn.Parameter(torch.empty(bias_len, **kw))
        elif bias:
            self.register_buffer("bias", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        # the weight dimension that is split over the workers: out channels are dim 0 of a
        # convolution kernel and dim 1 of a transposed one, in channels the other way round
        self.split_dim = 0 if (self.shard == "out") != self.transposed else 1
        self._register_state_dict_hook(self.gather_state_dict)
        self._register_load_state_dict_pre_hook(self.scatter_state_dict)
        if collect_state:
            self.P_root = root_partition(P_x)
            self.gather_weight = Repartition(self.P_weight, self.P_root, preserve_batch=False)
            self.scatter_weight = Repartition(self.P_root, self.P_weight, preserve_batch=False)
            if bias and self.shard == "out":
                self.gather_bias = Repartition(self.P_weight, self.P_root, preserve_batch=False)
                self.scatter_bias = Repartition(self.P_root, self.P_weight, preserve_batch=False)

    def _to_grid(self, w):
        """Puts the split dimension of a kernel where ``P_weight = [1, M, 1, ...]`` splits."""
        return w.transpose(0, 1).contiguous() if self.split_dim == 0 and w.dim() > 1 else w

    def gather_state_dict(self, module, destination, prefix, *args):
        """``collect_state=True``: the whole kernel (PyTorch layout) and bias on the first worker
        only (``src/distdl/nn/conv_channel_ag.py:264-300``)."""
        if not (getattr(self, "collect_state", False) and self.P_x.active):
            return destination
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        bias = destination.pop(bias_key, None)
        if self.use_bias and self.shard == "out" and self.P_weight.active:
            shape = [1] * self.P_x.dim
            shape[1] = -1
            bias = self.gather_bias(bias.detach().reshape(shape))
        weight = destination.pop(weight_key).detach()
        if self.P_weight.active:
            weight = self.gather_weight(self._to_grid(weight))
        if self.P_root.active:
            destination[weight_key] = self._to_grid(weight).contiguous()
            if self.use_bias:
                destination[bias_key] = bias.detach().reshape(-1)
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (getattr(self, "collect_state", False) and self.P_x.active):
            return destination
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        dev, dt = self._device, self.weight.dtype
        weight, bias = destination.pop(weight_key, None), destination.pop(bias_key, None)
        weight = self._to_grid(weight.to(dev)) if self.P_root.active else zero_volume_tensor(device=dev, dtype=dt)
        if self.P_weight.active:
            weight = self._to_grid(self.scatter_weight(weight)).contiguous()
        destination[weight_key] = weight
        if self.use_bias:
            if self.shard == "out":
                shape = [1] * self.P_x.dim
                shape[1] = -1
                bias = bias.to(dev).reshape(shape) if self.P_root.active else zero_volume_tensor(device=dev, dtype=dt)
                if self.P_weight.active:
                    bias = self.scatter_bias(bias).reshape(-1)
            elif not self.P_root.active:
                bias = zero_volume_tensor(device=dev, dtype=dt)
            else:
                bias = bias.to(dev)
            destination[bias_key] = bias
        return destination

    def extra_repr(self):
        return (f"{self.in_channels}, {self.out_channels}, kernel_size={self.kernel_size}, stride={self.stride}, "
                f"padding={self.padding}, dilation={self.dilation}, groups={self.groups}, bias={self.use_bias}")

    def reset_parameters(self):
        fan_in = (self.out_channels if self.transposed else self.in_channels) // self.groups * \
            int(np.prod(self.kernel_size))
        bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
        with torch.no_grad():
            if self.P_weight.active:
                self.weight.uniform_(-bound, bound)
            if self.use_bias and self.P_bias.active:
                self.bias.uniform_(-bound, bound)

    def _conv(self, x, w, b):
        nd = self.num_dimensions
        if self.transposed:
            return _CONVT[nd](x, w, b, stride=self.stride, padding=self.padding, output_padding=self.output_padding,
                              groups=self.groups, dilation=self.dilation)
        return _CONV[nd](x, w, b, stride=self.stride, padding=self.padding, dilation=self.dilation,
                         groups=self.groups)


class _ChannelAllGatherConv(_ChannelConvNd):
    r"""Weight split over its *output* channels on ``P_weight = [1, M, 1, ...]``
    (first data-parallel row), broadcast over the data-parallel workers; the
    input ``[batch/D, in/M, ...]`` is all-gathered along the channel dimension;
    the output is ``[batch/D, out/M, ...]``."""

    shard = "out"

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        if not self.P_x.active:
            return
        self.all_gather = AllGather(self.P_x, axes_all_gather=(1,))
        self.broadcast_bias = Broadcast(self.P_weight, self.P_x, preserve_batch=False) if self.use_bias else None

    def forward(self, input):
        if not self.P_x.active:
            return input
        w = self.broadcast_weight(self.weight)
        b = self.broadcast_bias(self.bias) if self.use_bias else None
        x = self.all_gather(input)
        return self._conv(x, w, b)


def _make(base, nd, transposed, name, doc):
    return type(name, (base,), {"num_dimensions": nd, "transposed": transposed, "__doc__": doc,
                                "__module__": base.__module__})


_DOC = "Channel all-gather {}convolution, {}-D (see the base class)."
for _nd in (1, 2, 3):
    for _transposed in (False, True):
        _name = f"DistributedChannelAllGatherConv{'Transpose' if _transposed else ''}{_nd}d"
        globals()[_name] = _make(_ChannelAllGatherConv, _nd, _transposed, _name,
                                 _DOC.format("transposed " if _transposed else "", _nd))
del _nd, _transposed, _name
