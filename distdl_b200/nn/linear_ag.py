"""Column-parallel linear layer: all-gather of the input, then a local GEMM.
Counterpart of ``src/distdl/nn/linear_ag.py:19-486``."""
import math

import numpy as np
import torch

from .. import ops
from ..utilities.torch import zero_volume_tensor
from . import init
from ._linear_common import PrefetchStream, derived_partition, local_out_features, relayout, root_partition, var_blocks
from .all_gather import AllGather
from .broadcast import Broadcast
from .module import Module
from .repartition import Repartition


class DistributedLinearAllGather(Module):
    r"""``y = x W^T + b`` with ``W`` split over its *output* features.

    ``P_y`` has shape ``[D, ..., 1, M]``: ``D`` data-parallel workers times ``M``
    tensor-parallel workers; the output is feature-sharded over ``M``.  The
    input lives on ``P_x`` (default ``P_y``: feature-sharded; ``[D, ..., M, 1]``:
    sequence-sharded, i.e. sequence parallelism) and is all-gathered along the
    sharded one of its last two dimensions before the GEMM.

    The weight ``[1, ..., out/M, in]`` (and bias ``[1, ..., out/M, 1]``) is
    stored on the first data-parallel row only (``P_store_weight``
    ``[1, ..., M, 1]``) and broadcast to the others every forward, so that
    data parallelism needs no separate gradient all-reduce: the adjoint of the
    broadcast sum-reduces the weight gradients onto the owners.

    ``collect_state=True`` makes ``state_dict()`` deliver the full weight in
    the serial ``torch.nn.Linear`` layout on the root worker (fused QKV / GQA /
    GEGLU blocks are de-interleaved with ``num_heads``, ``num_heads_kv``,
    ``num_vars``, ``geglu``), and ``load_state_dict`` accept it on any worker count.
    """

    def __init__(self, P_y, in_features, out_features, bias=True, device=None, dtype=None, P_x=None,
                 P_store_weight=None, P_apply_weight=None, collect_state=False, num_heads=None,
                 num_heads_kv=None, num_vars=3, geglu=False, scale_backward=None):
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
        self.use_bias = bias
        self.dtype = dtype
        dim, M = P_y.dim, int(P_y.shape[-1])
        if P_store_weight is None:
            idx = [slice(0, 1)] * dim
            idx[-1] = slice(0, M)
            shape = [1] * dim
            shape[-2] = M
            P_store_weight = derived_partition(P_y, idx, shape)
        if P_apply_weight is None:
            shape = [int(s) for s in P_y.shape]
            shape[-1], shape[-2] = 1, M
            P_apply_weight = P_y.create_partition_inclusive(range(P_y.size)).create_cartesian_topology_partition(shape)
        self.P_store_weight, self.P_apply_weight = P_store_weight, P_apply_weight
        self.broadcast_weight = Broadcast(P_store_weight, P_apply_weight, scale_backward=scale_backward)
        if bias:
            self.broadcast_bias = Broadcast(P_store_weight, P_apply_weight, scale_backward=scale_backward)
        tp_index = int(P_apply_weight.index[-2])
        self.out_features_local = local_out_features(out_features, M, tp_index, num_heads, num_heads_kv, num_vars,
                                                     geglu)
        if P_store_weight.active:
            wshape = [1] * dim
            wshape[-2], wshape[-1] = self.out_features_local, in_features
            self.weight = torch.nn.Parameter(torch.empty(tuple(wshape), **kw))
            if bias:
                bshape = [1] * dim
                bshape[-2] = self.out_features_local
                self.bias = torch.nn.Parameter(torch.empty(tuple(bshape), **kw))
            else:
                self.register_parameter("bias", None)
        else:
            self.register_buffer("weight", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
            if bias:
                self.register_buffer("bias", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
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
        if collect_state:
            self.P_root = root_partition(P_y)
            self.gather_weight = Repartition(P_store_weight, self.P_root, preserve_batch=False)
            self.scatter_weight = Repartition(self.P_root, P_store_weight, preserve_batch=False)
            if bias:
                self.gather_bias = Repartition(P_store_weight, self.P_root, preserve_batch=False)
                self.scatter_bias = Repartition(self.P_root, P_store_weight, preserve_batch=False)

    def reset_parameters(self):
        if self.P_store_weight.active:
            init.kaiming_uniform_(self.P_store_weight, self.weight, a=math.sqrt(5))
            if self.bias is not None:
                bound = 1 / math.sqrt(self.in_features) if self.in_features > 0 else 0
                init.uniform_(self.bias, -bound, bound)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.use_bias}"

    # ------------------------------------------------ serial <-> parallel layout
    def _blocks(self):
        return var_blocks(self.out_features, int(self.P_store_weight.shape[-2]), self.num_heads, self.num_heads_kv,
                          self.num_vars, self.geglu)

    def qkv_weight_to_serial(self, weight):
        return relayout(weight, weight.dim() - 2, self._blocks(), True)

    def qkv_weight_to_parallel(self, weight):
        return relayout(weight, weight.dim() - 2, self._blocks(), False)

    geglu_weight_to_serial = qkv_weight_to_serial
    geglu_weight_to_parallel = qkv_weight_to_parallel

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (self.collect_state and self.P_y.active):
            return destination
        if self.use_bias:
            bias_key = next(reversed(destination))
            bias = self.gather_bias(destination.pop(bias_key))
        weight_key = next(reversed(destination))
        weight = self.gather_weight(destination.pop(weight_key))
        if self.P_root.active:
            destination[weight_key] = self.qkv_weight_to_serial(weight).reshape(self.out_features, self.in_features)
            if self.use_bias:
                destination[bias_key] = self.qkv_weight_to_serial(bias).reshape(self.out_features)
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (self.collect_state and self.P_y.active):
            return destination
        dim = self.P_y.dim
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        weight = destination.pop(weight_key, None)
        if self.P_root.active:
            shape = [1] * dim
            shape[-2], shape[-1] = self.out_features, self.in_features
            weight = self.qkv_weight_to_parallel(weight.reshape(shape).to(self.P_y.device))
        else:
            weight = zero_volume_tensor(device=self.P_y.device, dtype=self.dtype)
        weight = self.scatter_weight(weight)
        bias = None
        if self.use_bias:
            bias = destination.pop(bias_key, None)
            if self.P_root.active:
                shape = [1] * dim
                shape[-2] = self.out_features
                bias = self.qkv_weight_to_parallel(bias.reshape(shape).to(self.P_y.device))
            else:
                bias = zero_volume_tensor(device=self.P_y.device, dtype=self.dtype)
            bias = self.scatter_bias(bias)
        destination[weight_key] = weight
        if self.use_bias:
            destination[bias_key] = bias
        return destination

    # ---------------------------------------------------------------- forward
    def prefetch_weights(self):
        """Starts the data-parallel weight broadcast on a side stream."""
        if self.P_y.size == 1:
            return

        def work():
            self.weight_buffer = self.broadcast_weight(self.weight).view(-1, self.in_features)
            if self.bias is not None:
                self.bias_buffer = self.broadcast_bias(self.bias).view(-1)
        self.prefetch.run(work)

    def forward(self, input):
        if not self.P_y.active:
            return input
        if self.weight_buffer is None:
            weight = self.broadcast_weight(self.weight).view(-1, self.in_features)
            bias = self.broadcast_bias(self.bias).view(-1) if self.bias is not None else None
        else:
            self.prefetch.wait()
            weight, bias = self.weight_buffer, self.bias_buffer
            self.weight_buffer = self.bias_buffer = None
        fused = _fused_ag_linear(self, input, weight, bias)
        if fused is not None:
            return fused
        input = self.all_gather(input)
        return ops.linear(input, weight, bias)


def _fused_ag_linear(layer, input, weight, bias):
    """all-gather -> GEMM in one kernel (native backend, CUDA, sequence- or
    feature-sharded bf16 input); ``None`` when the fused path does not apply."""
    if not input.is_cuda or getattr(layer._distdl_backend, "name", "") != "native_cupy":
        return None
    from ..parallel import fused
    return fused.maybe_ag_linear(layer, input, weight, bias)
