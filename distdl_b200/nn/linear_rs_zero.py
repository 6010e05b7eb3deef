"""Row-parallel linear layer with ZeRO-3 / FSDP weight sharding.
Counterpart of ``src/distdl/nn/linear_rs_zero.py:20-471``."""
import math

import numpy as np
import torch

from .. import ops
from ..utilities import recompute
from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import (KeptBufferGuard, PrefetchStream, deliver_grad, derived_partition, direct_main_grad,
                             reduce_scatter_grad, root_partition)
from .all_gather import AllGather
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


class DistributedLinearReduceScatterZero(Module):
    r"""``y = x W^T + b`` with ``W`` split over its input features across the
    ``M`` tensor-parallel workers and over its output features across the ``D``
    data-parallel workers.

    ``P_x = [D, ..., 1, M]``; weight shard ``[out/D, 1, ..., in/M]`` lives on
    ``P_x`` itself; bias shard ``[out/D, 1, ...]`` on ``P_bias = [D, ..., 1, 1]``
    (first tensor-parallel column, so the bias enters the reduction once).
    Forward: all-gather the weight over ``D``, local GEMM, reduce-scatter of the
    partial products over ``M`` (along features, or along the sequence when
    ``P_y = [D, ..., M, 1]``).  ``checkpoint`` and ``auto_clear_buffer`` behave
    as in :class:`DistributedLinearAllGatherZero`.
    """

    def __init__(self, P_x, in_features, out_features, bias=True, device=None, dtype=None, P_y=None,
                 P_bias=None, collect_state=False, checkpoint=False, scale_backward=None, auto_clear_buffer=True,
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
        self.checkpoint, self.scale_backward, self.auto_clear_buffer = checkpoint, scale_backward, auto_clear_buffer
        dim, M, D = P_x.dim, int(P_x.shape[-1]), int(P_x.shape[0])
        if bias and P_bias is None:
            idx = [slice(0, int(s)) for s in P_x.shape]
            idx[-1] = slice(0, 1)
            shape = [int(s) for s in P_x.shape]
            shape[-1] = 1
            P_bias = derived_partition(P_x, idx, shape)
        self.P_bias = P_bias if bias else None
        self.allgather_weight = AllGather(P_x, axes_all_gather=(0,), scale_backward=scale_backward)
        self.reduce_scatter_weight = ReduceScatter(P_x, axes_reduce_scatter=(0,))
        wshape = [1] * dim
        wshape[0] = int(compute_subshape(D, P_x.index[0], [out_features])[0])
        wshape[-1] = _local_in(in_features, M, int(P_x.index[-1]), num_heads)
        self.in_features_local = wshape[-1]
        self.weight = torch.nn.Parameter(torch.empty(tuple(wshape), **kw))
        # lets an optimizer find the all-gather of this ZeRO shard (team, gathered layout)
        self.weight.zero_gather = self.allgather_weight
        self._kept = KeptBufferGuard()
        if bias and self.P_bias.active:
            self.allgather_bias = AllGather(self.P_bias, axes_all_gather=(0,), scale_backward=scale_backward)
            self.reduce_scatter_bias = ReduceScatter(self.P_bias, axes_reduce_scatter=(0,))
            bshape = [1] * dim
            bshape[0] = wshape[0]
            self.bias = torch.nn.Parameter(torch.empty(tuple(bshape), **kw))
        elif bias:
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
        self.P_root = root_partition(P_x)
        # weight [out/D, 1.., in/M] is laid out over P_x as (dim0 = D, last = M)
        self.gather_weight = Repartition(P_x, self.P_root, preserve_batch=False)
        self.scatter_weight = Repartition(self.P_root, P_x, preserve_batch=False)
        if bias:
            self.gather_bias = Repartition(self.P_bias, self.P_root, preserve_batch=False)
            self.scatter_bias = Repartition(self.P_root, self.P_bias, preserve_batch=False)

    def reset_parameters(self):
        bound = 1 / math.sqrt(self.in_features) if self.in_features > 0 else 0
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)
            if self.use_bias and self.P_bias.active:
                self.bias.uniform_(-bound, bound)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.use_bias}"

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        weight = self.gather_weight(destination.pop(weight_key).detach())
        bias = None
        if self.use_bias:
            b = destination.pop(bias_key)
            bias = self.gather_bias(b.detach() if self.P_bias.active else
                                    zero_volume_tensor(device=self.P_x.device, dtype=self.dtype))
        if self.P_root.active:
            destination[weight_key] = weight.reshape(self.out_features, self.in_features)
            if self.use_bias:
                destination[bias_key] = bias.reshape(self.out_features)
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        dim = self.P_x.dim
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        weight = destination.pop(weight_key, None)
        if self.P_root.active:
            shape = [1] * dim
            shape[0], shape[-1] = self.out_features, self.in_features
            weight = weight.reshape(shape).to(self.P_x.device)
        else:
            weight = zero_volume_tensor(device=self.P_x.device, dtype=self.dtype)
        destination[weight_key] = self.scatter_weight(weight)
        if self.use_bias:
            bias = destination.pop(bias_key, None)
            if self.P_root.active:
                shape = [1] * dim
                shape[0] = self.out_features
                bias = bias.reshape(shape).to(self.P_x.device)
            else:
                bias = zero_volume_tensor(device=self.P_x.device, dtype=self.dtype)
            destination[bias_key] = self.scatter_bias(bias)
        return destination

    def _collect_weights(self):
        w = self.allgather_weight(self.weight)                 # [out, 1.., in/M]
        self.weight_buffer = w.reshape(self.out_features, self.in_features_local)
        if self.use_bias and self.P_bias.active:
            self.bias_buffer = self.allgather_bias(self.bias).reshape(self.out_features)
        if not self.auto_clear_buffer:
            self.weight_buffer = self.weight_buffer.detach().requires_grad_(True)
            if self.bias_buffer is not None:
                self.bias_buffer = self.bias_buffer.detach().requires_grad_(True)

    def collect_weights(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        bias = self.bias if (self.use_bias and self.P_bias.active) else None
        if self.weight_buffer is not None and not self.auto_clear_buffer and self._kept.stale(self.weight, bias):
            self.weight_buffer = self.bias_buffer = None
        if self.weight_buffer is None:
            self.prefetch.run(self._collect_weights)
            self._kept.remember(self.weight, bias)

    prefetch_weights = collect_weights

    def wait_for_streams(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        self.prefetch.wait()

    def clear_weight_buffer(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if not self.auto_clear_buffer and self.weight_buffer is not None and self.weight_buffer.grad is not None:
            g = self.weight_buffer.grad
            reduce_scatter_grad(self.reduce_scatter_weight, g.reshape([self.out_features] + list(self.weight.shape[1:])),
                                self.weight, self.scale_backward)
            if self.bias_buffer is not None and self.bias_buffer.grad is not None:
                gb = self.bias_buffer.grad
                if self.scale_backward is not None:
                    gb = gb / self.scale_backward
                gbl = self.reduce_scatter_bias(gb.reshape([self.out_features] + [1] * (self.P_x.dim - 1)))
                deliver_grad(self.bias, gbl)
        self.weight_buffer = None
        self.bias_buffer = None

    def _linear_then_scatter(self, input, w, b):
        if input.is_cuda and getattr(self._distdl_backend, "name", "") == "native_cupy":
            from ..parallel import fused
            y = fused.maybe_linear_rs(self, input, w, b)
            if y is not None:
                return y
        y = ops.linear(input, w, b)
        return self.reduce_scatter(y)

    def forward(self, input):
        if not self.P_x.active:
            return input
        if self.checkpoint:
            bias = self.bias if (self.use_bias and self.P_bias.active) else None
            return _CheckpointedRSZero.apply(self, input, self.weight, bias)
        self.collect_weights()
        self.wait_for_streams()
        w = self.weight_buffer
        base = w
        mg = direct_main_grad(self.weight, self.allgather_weight, w.shape)
        if mg is not None:
            w = w.view(w.shape)              # a fresh tensor object to carry the attribute
            w.main_grad = mg
        # where recipes are on, the backward pass gathers the weight shards again instead of
        # holding the gathered weight since the forward pass
        resharded = self.auto_clear_buffer and int(self.allgather_weight.P_x.shape[self.allgather_weight.axes_all_gather[0]]) > 1
        with recompute.saved_as_recipe(base, self._regather if resharded else None):
            y = self._linear_then_scatter(input, w, self.bias_buffer)
        if self.auto_clear_buffer:
            self.clear_weight_buffer()
        return y

    def _regather(self):
        """The gathered weight ``[out, in/M]`` once more, for the backward pass (taken from a
        prefetch if one is pending)."""
        self.collect_weights()
        self.wait_for_streams()
        w = self.weight_buffer
        if self.auto_clear_buffer:
            self.weight_buffer = self.bias_buffer = None
        return w


class _CheckpointedRSZero(torch.autograd.Function):
    """Saves the sharded operands and re-gathers the weight in backward
    (``src/distdl/nn/linear_rs_zero.py:20-82``)."""

    @staticmethod
    def forward(ctx, layer, input, weight, bias):
        ctx.layer = layer
        ctx.save_for_backward(input, weight, bias)
        with torch.no_grad():
            w = layer.allgather_weight(weight).reshape(layer.out_features, layer.in_features_local)
            b = layer.allgather_bias(bias).reshape(layer.out_features) if bias is not None else None
            return layer._linear_then_scatter(input, w, b)

    @staticmethod
    def backward(ctx, grad_output):
        layer = ctx.layer
        input, weight, bias = ctx.saved_tensors
        with torch.enable_grad():
            xi = input.detach().requires_grad_(input.requires_grad)
            wi = weight.detach().requires_grad_(True)
            bi = bias.detach().requires_grad_(True) if bias is not None else None
            w = layer.allgather_weight(wi).reshape(layer.out_features, layer.in_features_local)
            b = layer.allgather_bias(bi).reshape(layer.out_features) if bi is not None else None
            y = layer._linear_then_scatter(xi, w, b)
        ins = [t for t in (xi, wi, bi) if t is not None and t.requires_grad]
        grads = iter(torch.autograd.grad(y, ins, grad_output))
        gx = next(grads) if xi.requires_grad else None
        gw = next(grads)
        gb = next(grads) if bi is not None else None
        return None, gx, gw, gb
