"""Column-parallel linear layer with ZeRO-3 / FSDP weight sharding.
Counterpart of ``src/distdl/nn/linear_ag_zero.py:21-622``."""
import math

import numpy as np
import torch

from .. import ops
from ..utilities import recompute
from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import (KeptBufferGuard, PrefetchStream, deliver_grad, direct_main_grad, local_out_features,
                             reduce_scatter_grad, relayout, root_partition, var_blocks)
from .all_gather import AllGather
from .module import Module
from .reduce_scatter import ReduceScatter
from .repartition import Repartition


class DistributedLinearAllGatherZero(Module):
    r"""``y = x W^T + b`` with ``W`` split over its output features across the
    ``M`` tensor-parallel workers *and* over its input features across the
    ``D`` data-parallel workers (fully sharded data parallelism).

    ``P_y = [D, ..., 1, M]``; weight shard ``[in/D, 1, ..., out/M, 1]`` on
    ``P_weight = [D, ..., M, 1]``; bias shard ``[1, ..., out/M/D, 1]``.  Each
    forward all-gathers the weight shards over ``D`` (:meth:`collect_weights`,
    optionally ahead of time on a side stream), all-gathers the input over ``M``
    and runs the local GEMM; autograd reduce-scatters the weight gradients back
    onto the shards.  ``checkpoint=True`` saves only the *sharded* operands and
    re-gathers them in backward.  ``auto_clear_buffer=False`` keeps the gathered
    weights across micro-batches (ZeRO-1 style): their gradients accumulate
    locally and :meth:`clear_weight_buffer` reduce-scatters them once.

    The gathered weight ``[in, out/M]`` feeds the GEMM as an MN-major operand;
    no transposed copy is made.
    """

    def __init__(self, P_y, in_features, out_features, bias=True, device=None, dtype=None, P_x=None,
                 P_store_bias=None, P_weight=None, collect_state=False, num_heads=None, num_heads_kv=None,
                 num_vars=3, geglu=False, checkpoint=False, scale_backward=None, auto_clear_buffer=True):
        super().__init__()
        self.P_y = P_y
        if not P_y.active:
            return
        assert P_y.shape[-2] == 1
        if P_x is None:
            self.P_x = P_y
        else:
            assert P_x.dim == P_y.dim and P_x.shape[-2] == P_y.shape[-1] and P_x.shape[-1] == 1
            self.P_x = P_x
        device = device if device is not None else P_y.device
        kw = {"device": device, "dtype": dtype}
        self.in_features, self.out_features = in_features, out_features
        self.collect_state = collect_state
        self.num_heads, self.num_heads_kv, self.num_vars, self.geglu = num_heads, num_heads_kv, num_vars, geglu
        self.use_bias, self.dtype = bias, dtype
        self.checkpoint, self.scale_backward, self.auto_clear_buffer = checkpoint, scale_backward, auto_clear_buffer
        dim, M = P_y.dim, int(P_y.shape[-1])
        if P_weight is None:
            shape = [int(s) for s in P_y.shape]
            shape[-1], shape[-2] = 1, M
            P_weight = P_y.create_partition_inclusive(range(P_y.size)).create_cartesian_topology_partition(shape)
        self.P_weight = P_weight
        if P_store_bias is not None:
            # the partition [1, ..., M, 1] through which the bias travels between its shards and the
            # serial state dict (``src/distdl/nn/linear_ag_zero.py:202-207``): member j must be a worker
            # of tensor-parallel column j, since it contributes that column's bias slice
            assert P_store_bias.dim == P_y.dim and int(P_store_bias.shape[-1]) == 1
            assert int(P_store_bias.shape[-2]) == M
            assert int(np.prod(P_store_bias.shape[:dim - 2])) == 1
            if P_store_bias.active and int(P_store_bias.index[-2]) != int(P_weight.index[-2]):
                raise ValueError("P_store_bias: member j must belong to tensor-parallel column j of P_weight")
        self.P_store_bias = P_store_bias
        D = int(P_weight.shape[0])
        self.allgather_weight = AllGather(P_weight, axes_all_gather=(0,), scale_backward=scale_backward)
        self.reduce_scatter_weight = ReduceScatter(P_weight, axes_reduce_scatter=(0,))
        tp_index = int(P_weight.index[-2])
        self.out_features_local = local_out_features(out_features, M, tp_index, num_heads, num_heads_kv, num_vars,
                                                     geglu)
        wshape = [1] * dim
        wshape[0] = int(compute_subshape(D, P_weight.index[0], [in_features])[0])
        wshape[-2] = self.out_features_local
        self.weight = torch.nn.Parameter(torch.empty(tuple(wshape), **kw))
        # lets an optimizer find the all-gather of this ZeRO shard (team, gathered layout)
        self.weight.zero_gather = self.allgather_weight
        self._kept = KeptBufferGuard()
        if bias:
            bshape = [1] * dim
            bshape[-2] = int(compute_subshape(D, P_weight.index[0], [self.out_features_local])[0])
            self.bias = torch.nn.Parameter(torch.empty(tuple(bshape), **kw))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        gather_dim = int(np.argmax(np.asarray(self.P_x.shape[-2:]))) + dim - 2
        self.gather_dim = gather_dim
        self.all_gather = AllGather(self.P_x, axes_all_gather=(gather_dim,))
        self.prefetch = PrefetchStream(device)
        self.weight_buffer = None
        self.bias_buffer = None
        self._register_state_dict_hook(self.gather_state_dict)
        self._register_load_state_dict_pre_hook(self.scatter_state_dict)
        self.P_root = root_partition(P_y)
        self.gather_weight = Repartition(P_weight, self.P_root, preserve_batch=False)
        self.scatter_weight = Repartition(self.P_root, P_weight, preserve_batch=False)

    def reset_parameters(self):
        bound = 1 / math.sqrt(self.in_features) if self.in_features > 0 else 0
        with torch.no_grad():
            # kaiming_uniform(a=sqrt(5)) on a [out, in] weight == U(-1/sqrt(in), 1/sqrt(in))
            self.weight.uniform_(-bound, bound)
            if self.bias is not None:
                self.bias.uniform_(-bound, bound)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.use_bias}"

    # ------------------------------------------------------------ state dicts
    def _blocks(self):
        return var_blocks(self.out_features, int(self.P_weight.shape[-2]), self.num_heads, self.num_heads_kv,
                          self.num_vars, self.geglu)

    def qkv_weight_to_serial(self, weight):
        return relayout(weight, weight.dim() - 2, self._blocks(), True)

    def qkv_weight_to_parallel(self, weight):
        return relayout(weight, weight.dim() - 2, self._blocks(), False)

    geglu_weight_to_serial = qkv_weight_to_serial
    geglu_weight_to_parallel = qkv_weight_to_parallel

    def allgather_bias_over_dp(self, bias):
        """Bias shards -> the whole tensor-parallel bias slice ``[1, ..., out/M, 1]``: the
        feature dim is moved to dim 0 (the data-parallel partition dim), gathered, moved back."""
        return self._bias_ag(bias.transpose(0, -2)).transpose(0, -2)

    @property
    def _bias_ag(self):
        if not hasattr(self, "_bias_ag_module"):
            object.__setattr__(self, "_bias_ag_module",
                               AllGather(self.P_weight, axes_all_gather=(0,), scale_backward=self.scale_backward))
        return self._bias_ag_module

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (self.collect_state and self.P_y.active):
            return destination
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        if self.use_bias:
            bias = self.allgather_bias_over_dp(destination.pop(bias_key).detach())   # [1,..,out/M,1] per TP column
            full = self._gather_tp(bias)
        weight = self.gather_weight(destination.pop(weight_key).detach())
        if self.P_root.active:
            w = self.qkv_weight_to_serial(weight)                       # [in, 1.., out, 1]
            destination[weight_key] = w.reshape(self.in_features, self.out_features).t().contiguous()
            if self.use_bias:
                destination[bias_key] = self.qkv_weight_to_serial(full).reshape(self.out_features)
        return destination

    def _gather_tp(self, bias_col):
        """Concatenates the per-column bias slices over the tensor-parallel dim onto the root."""
        if not hasattr(self, "_bias_gather"):
            dim = self.P_y.dim
            idx = [slice(0, 1)] * dim
            idx[-2] = slice(0, int(self.P_weight.shape[-2]))
            shape = [1] * dim
            shape[-2] = int(self.P_weight.shape[-2])
            from ._linear_common import derived_partition
            P_col = self.P_store_bias if self.P_store_bias is not None else derived_partition(self.P_weight, idx, shape)
            object.__setattr__(self, "_P_bias_col", P_col)
            object.__setattr__(self, "_bias_gather", Repartition(P_col, self.P_root, preserve_batch=False))
            object.__setattr__(self, "_bias_scatter", Repartition(self.P_root, P_col, preserve_batch=False))
        x = bias_col if self._P_bias_col.active else zero_volume_tensor(device=bias_col.device, dtype=bias_col.dtype)
        return self._bias_gather(x)

    def scatter_state_dict(self, destination, prefix, *args):
        if not (self.collect_state and self.P_y.active):
            return destination
        dim = self.P_y.dim
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        weight = destination.pop(weight_key, None)
        if self.P_root.active:
            shape = [1] * dim
            shape[0], shape[-2] = self.in_features, self.out_features
            weight = self.qkv_weight_to_parallel(weight.t().reshape(shape).to(self.P_y.device))
        else:
            weight = zero_volume_tensor(device=self.P_y.device, dtype=self.dtype)
        destination[weight_key] = self.scatter_weight(weight)
        if self.use_bias:
            bias = destination.pop(bias_key, None)
            self._gather_tp(self.allgather_bias_over_dp(self.bias.detach()))  # builds the helper partitions
            if self.P_root.active:
                shape = [1] * dim
                shape[-2] = self.out_features
                bias = self.qkv_weight_to_parallel(bias.reshape(shape).to(self.P_y.device))
            else:
                bias = zero_volume_tensor(device=self.P_y.device, dtype=self.dtype)
            col = self._bias_scatter(bias)      # [1,..,out/M,1] on data-parallel row 0, zero-volume elsewhere
            from .broadcast import Broadcast
            if not hasattr(self, "_bias_bcast"):
                object.__setattr__(self, "_bias_bcast", Broadcast(self._P_bias_col, self.P_weight,
                                                                  preserve_batch=False))
            col = self._bias_bcast(col)
            D, d = int(self.P_weight.shape[0]), int(self.P_weight.index[0])
            n = col.shape[-2]
            lo = (n // D) * d + min(d, n % D)
            destination[bias_key] = col.narrow(dim - 2, lo, self.bias.shape[-2]).contiguous()
        return destination

    # ---------------------------------------------------------------- forward
    def _collect_weights(self):
        w = self.allgather_weight(self.weight)            # [in, 1.., out/M, 1]
        self.weight_buffer = w.reshape(self.in_features, self.out_features_local)
        if self.bias is not None:
            self.bias_buffer = self.allgather_bias_over_dp(self.bias).reshape(self.out_features_local)
        if not self.auto_clear_buffer:
            # ZeRO-1 mode: the gathered tensors become leaves that accumulate gradients
            self.weight_buffer = self.weight_buffer.detach().requires_grad_(True)
            if self.bias is not None:
                self.bias_buffer = self.bias_buffer.detach().requires_grad_(True)

    def collect_weights(self):
        """Gathers the weight (and bias) shards, on the side stream when there is one."""
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if self.weight_buffer is not None and not self.auto_clear_buffer and self._kept.stale(self.weight, self.bias):
            self.weight_buffer = self.bias_buffer = None
        if self.weight_buffer is None:
            self.prefetch.run(self._collect_weights)
            self._kept.remember(self.weight, self.bias)

    prefetch_weights = collect_weights

    def wait_for_streams(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        self.prefetch.wait()

    def clear_weight_buffer(self):
        """Drops the gathered weights.  In ZeRO-1 mode first reduce-scatters the
        gradients accumulated on them into ``weight.grad`` / ``bias.grad``."""
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if not self.auto_clear_buffer and self.weight_buffer is not None and self.weight_buffer.grad is not None:
            g = self.weight_buffer.grad
            reduce_scatter_grad(self.reduce_scatter_weight, g.reshape([self.in_features] + list(self.weight.shape[1:])),
                                self.weight, self.scale_backward)
            if self.bias is not None and self.bias_buffer.grad is not None:
                gb = self.bias_buffer.grad
                if self.scale_backward is not None:
                    gb = gb / self.scale_backward
                shape = [1] * self.P_y.dim
                shape[0] = self.out_features_local
                if not hasattr(self, "_bias_rs"):
                    object.__setattr__(self, "_bias_rs", ReduceScatter(self.P_weight, axes_reduce_scatter=(0,)))
                gbl = self._bias_rs(gb.reshape(shape)).transpose(0, -2)
                deliver_grad(self.bias, gbl)
        self.weight_buffer = None
        self.bias_buffer = None

    def forward(self, input):
        if not self.P_y.active:
            return input
        if self.checkpoint:
            return _CheckpointedAGZero.apply(self, input, self.weight, self.bias)
        self.collect_weights()
        self.wait_for_streams()
        w, b = self.weight_buffer, self.bias_buffer
        wt = w.t()
        mg = direct_main_grad(self.weight, self.allgather_weight, w.shape)
        if mg is not None:
            wt.main_grad = mg.t()
        y = None
        # where recipes are on, the backward pass gathers the weight shards again instead of
        # holding the gathered weight since the forward pass
        with recompute.saved_as_recipe(w, self._regather if self._resharded_between_passes() else None):
            if input.is_cuda and getattr(self._distdl_backend, "name", "") == "native_cupy":
                from ..parallel import fused
                y = fused.maybe_ag_linear(self, input, wt, b)
            if y is None:
                x = self.all_gather(input)
                y = ops.linear(x, wt, b)
        if self.auto_clear_buffer:
            self.clear_weight_buffer()
        return y

    def _resharded_between_passes(self):
        return self.auto_clear_buffer and int(self.P_weight.shape[0]) > 1

    def _regather(self):
        """The gathered weight ``[in, out/M]`` once more, for the backward pass (taken from a
        prefetch if one is pending)."""
        self.collect_weights()
        self.wait_for_streams()
        w = self.weight_buffer
        if self.auto_clear_buffer:
            self.weight_buffer = self.bias_buffer = None
        return w


class _CheckpointedAGZero(torch.autograd.Function):
    """Saves the *sharded* input and weight; backward re-gathers both
    (``src/distdl/nn/linear_ag_zero.py:21-77``)."""

    @staticmethod
    def forward(ctx, layer, input, weight, bias):
        ctx.layer = layer
        ctx.save_for_backward(input, weight, bias)
        with torch.no_grad():
            w = layer.allgather_weight(weight).reshape(layer.in_features, layer.out_features_local)
            b = layer.allgather_bias_over_dp(bias).reshape(layer.out_features_local) if bias is not None else None
            x = layer.all_gather(input)
            return ops.linear(x, w.t(), b)

    @staticmethod
    def backward(ctx, grad_output):
        layer = ctx.layer
        input, weight, bias = ctx.saved_tensors
        with torch.enable_grad():
            xi = input.detach().requires_grad_(input.requires_grad)
            wi = weight.detach().requires_grad_(True)
            bi = bias.detach().requires_grad_(True) if bias is not None else None
            w = layer.allgather_weight(wi).reshape(layer.in_features, layer.out_features_local)
            b = layer.allgather_bias_over_dp(bi).reshape(layer.out_features_local) if bi is not None else None
            x = layer.all_gather(xi)
            y = ops.linear(x, w.t(), b)
        ins = [t for t in (xi, wi, bi) if t is not None and t.requires_grad]
        grads = torch.autograd.grad(y, ins, grad_output)
        it = iter(grads)
        gx = next(it) if xi.requires_grad else None
        gw = next(it)
        gb = next(it) if bi is not None else None
        return None, gx, gw, gb
