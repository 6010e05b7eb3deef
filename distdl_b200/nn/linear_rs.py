"""Row-parallel linear layer: local GEMM, then reduce-scatter of the partial
outputs.  Counterpart of ``src/distdl/nn/linear_rs.py:18-364``."""
import math

import numpy as np
import torch

from .. import ops
from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from . import init
from ._linear_common import PrefetchStream, derived_partition, root_partition
from .broadcast import Broadcast
from .module import Module
from .reduce_scatter import ReduceScatter
from .repartition import Repartition


def _local_in(in_features, M, index, num_heads):
    """Input features held by tensor-parallel worker ``index``: the balanced split, or --
    with ``num_heads`` -- a whole number of attention heads (so that it lines up with the
    per-worker output of a head-split QKV projection when heads do not divide evenly)."""
    if num_heads is None:
        return int(compute_subshape(M, index, [in_features])[0])
    return int(compute_subshape(M, index, [num_heads])[0]) * (in_features // num_heads)


class DistributedLinearReduceScatter(Module):
    r"""``y = x W^T + b`` with ``W`` split over its *input* features.

    ``P_x`` has shape ``[D, ..., 1, M]`` (input feature-sharded over the ``M``
    tensor-parallel workers).  Every worker multiplies its feature slice with
    its weight slice ``[1, ..., out, in/M]``; the partial products are
    reduce-scattered over ``M`` along the sharded one of the last two
    dimensions of ``P_y`` (default ``P_x``: features; ``[D, ..., M, 1]``:
    sequence, i.e. sequence-parallel output).  The bias lives on one worker and
    is added on the first tensor-parallel column only, so it enters the sum once.
    Weights are stored on the first data-parallel row and broadcast each forward.
    """

    def __init__(self, P_x, in_features, out_features, bias=True, device=None, dtype=None, P_y=None,
                 P_weight=None, P_store_bias=None, P_apply_bias=None, collect_state=False, scale_backward=None,
                 num_heads=None):
        super().__init__()
        self.P_x = P_x
        if not P_x.active:
            return
        assert P_x.shape[-2] == 1
        if P_y is None:
            self.P_y = P_x
        else:
            assert P_y.dim == P_x.dim and P_y.shape[-2] == P_x.shape[-1] and P_y.shape[-1] == 1
            self.P_y = P_y
        device = device if device is not None else P_x.device
        kw = {"device": device, "dtype": dtype}
        self.in_features, self.out_features = in_features, out_features
        self.collect_state, self.use_bias, self.dtype = collect_state, bias, dtype
        dim, M = P_x.dim, int(P_x.shape[-1])
        if P_weight is None:
            idx = [slice(0, 1)] * dim
            idx[-1] = slice(0, M)
            shape = [1] * dim
            shape[-1] = M
            P_weight = derived_partition(P_x, idx, shape)
        if bias and P_store_bias is None:
            P_store_bias = root_partition(P_x)
        if bias and P_apply_bias is None:
            idx = [slice(0, 1)] * dim
            for i in range(dim - 2):
                idx[i] = slice(0, int(P_x.shape[i]))
            shape = [int(s) for s in P_x.shape]
            shape[-2:] = [1, 1]
            P_apply_bias = derived_partition(P_x, idx, shape)
        self.P_weight = P_weight
        self.P_store_bias, self.P_apply_bias = (P_store_bias, P_apply_bias) if bias else (None, None)
        self.broadcast_weight = Broadcast(P_weight, P_x, scale_backward=scale_backward)
        if bias and self.P_apply_bias.active:
            self.broadcast_bias = Broadcast(P_store_bias, P_apply_bias, scale_backward=scale_backward)
        if P_weight.active:
            wshape = [1] * dim
            wshape[-1] = _local_in(in_features, M, int(P_weight.index[-1]), num_heads)
            wshape[-2] = out_features
            self.weight = torch.nn.Parameter(torch.empty(tuple(wshape), **kw))
        else:
            self.register_buffer("weight", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
        if bias and self.P_store_bias.active:
            bshape = [1] * dim
            bshape[-2] = out_features
            self.bias = torch.nn.Parameter(torch.empty(tuple(bshape), **kw))
        elif bias and self.P_apply_bias.active:
            self.register_buffer("bias", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        scatter_dim = int(np.argmax(np.asarray(self.P_y.shape[-2:]))) + dim - 2
        self.scatter_dim = scatter_dim
        self.reduce_scatter = ReduceScatter(self.P_y, axes_reduce_scatter=(scatter_dim,))
        self.prefetch = PrefetchStream(device)
        self.weight_buffer = None
        self.bias_buffer = None
        self._register_state_dict_hook(self.gather_state_dict)
        self._register_load_state_dict_pre_hook(self.scatter_state_dict)
        if collect_state:
            self.P_root = root_partition(P_x)
            self.gather_weight = Repartition(P_weight, self.P_root, preserve_batch=False)
            self.scatter_weight = Repartition(self.P_root, P_weight, preserve_batch=False)

    def reset_parameters(self):
        if self.P_weight.active:
            init.kaiming_uniform_(self.P_weight, self.weight, a=math.sqrt(5))
        if self.use_bias and self.P_store_bias.active:
            bound = 1 / math.sqrt(self.in_features) if self.in_features > 0 else 0
            init.uniform_(self.bias, -bound, bound)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.use_bias}"

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        weight_key = prefix + "weight"
        weight = self.gather_weight(destination.pop(weight_key))
        if self.P_root.active:
            destination[weight_key] = weight.reshape(self.out_features, self.in_features)
            if self.use_bias and (prefix + "bias") in destination:
                destination[prefix + "bias"] = destination[prefix + "bias"].reshape(self.out_features)
        elif self.use_bias:
            destination.pop(prefix + "bias", None)
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        dim = self.P_x.dim
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        weight = destination.pop(weight_key, None)
        if self.P_root.active:
            shape = [1] * dim
            shape[-2], shape[-1] = self.out_features, self.in_features
            weight = weight.reshape(shape).to(self.P_x.device)
        else:
            weight = zero_volume_tensor(device=self.P_x.device, dtype=self.dtype)
        destination[weight_key] = self.scatter_weight(weight)
        if self.use_bias:
            bias = destination.pop(bias_key, None)
            if self.P_store_bias.active:
                shape = [1] * dim
                shape[-2] = self.out_features
                destination[bias_key] = bias.reshape(shape).to(self.P_x.device)
            elif self.P_apply_bias.active:
                destination[bias_key] = zero_volume_tensor(device=self.P_x.device, dtype=self.dtype)
        return destination

    def prefetch_weights(self):
        if self.P_x.size == 1:
            return

        def work():
            self.weight_buffer = self.broadcast_weight(self.weight).view(self.out_features, -1)
            if self.bias is not None:
                self.bias_buffer = self.broadcast_bias(self.bias).view(self.out_features)
        self.prefetch.run(work)

    def forward(self, input):
        if not self.P_x.active:
            return input
        if self.weight_buffer is None:
            weight = self.broadcast_weight(self.weight).view(self.out_features, -1)
            bias = self.broadcast_bias(self.bias).view(self.out_features) if self.bias is not None else None
        else:
            self.prefetch.wait()
            weight, bias = self.weight_buffer, self.bias_buffer
            self.weight_buffer = self.bias_buffer = None
        fused = _fused_linear_rs(self, input, weight, bias)
        if fused is not None:
            return fused
        y = ops.linear(input, weight, bias)
        return self.reduce_scatter(y)


def _fused_linear_rs(layer, input, weight, bias):
    """GEMM -> reduce-scatter in one kernel (native backend, CUDA bf16)."""
    if not input.is_cuda or getattr(layer._distdl_backend, "name", "") != "native_cupy":
        return None
    from ..parallel import fused
    return fused.maybe_linear_rs(layer, input, weight, bias)
