"""Expert-parallel row-parallel linear layer
(``src/distdl/nn/linear_rs_expert.py:20-396``)."""
import math

import torch

from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import PrefetchStream, deliver_grad, derived_partition, root_partition
from .all_gather import AllGather
from .broadcast import Broadcast
from .linear_ag_expert import _expert_matmul
from .module import Module
from .reduce_scatter import ReduceScatter
from .repartition import Repartition


class DistributedExpertReduceScatter(Module):
    r"""Per-expert linear map whose *input* features are split over the ``M``
    tensor-parallel workers: ``P_expert_emb = [E, N, 1, M]``, weight shard
    ``[experts/E, out/N, in/M]`` on ``P_weight = [E, N, M]`` (ZeRO-sharded over
    ``N`` along the output features).  Forward: gather the weight over ``N``,
    grouped GEMM on the local feature slice, reduce-scatter of the partial
    outputs over ``M`` (features, or sequence with ``P_expert_seq = [E, N, S, 1]``).
    The bias ``[experts/E, 1, 1 -> out]`` is stored once per expert group and
    added on the first tensor-parallel column only.

    ``collect_state=True``: ``state_dict()`` holds, on the first worker only, the whole weight
    ``[experts, out, in]`` and bias ``[experts, 1, out]``; ``load_state_dict`` scatters that
    layout from the first worker (``src/distdl/nn/linear_rs_expert.py:253-298``)."""

    def __init__(self, P_expert_emb, num_experts, in_features, out_features, bias=True, device=None, dtype=None,
                 P_store_bias=None, P_apply_bias=None, P_weight=None, collect_state=False, scale_backward=None,
                 P_expert_seq=None, auto_clear_buffer=True):
        super().__init__()
        self.P_expert_emb, self.P_expert_seq = P_expert_emb, P_expert_seq
        if not P_expert_emb.active:
            return
        assert P_expert_emb.dim == 4
        device = device if device is not None else P_expert_emb.device
        kw = {"device": device, "dtype": dtype}
        self.num_experts, self.in_features, self.out_features = num_experts, in_features, out_features
        self.use_bias, self.collect_state = bias, collect_state
        self.scale_backward, self.auto_clear_buffer, self.dtype = scale_backward, auto_clear_buffer, dtype
        E, N, M = (int(P_expert_emb.shape[i]) for i in (0, 1, 3))
        if P_weight is None:
            P_weight = P_expert_emb.create_partition_inclusive(range(P_expert_emb.size)) \
                .create_cartesian_topology_partition([E, N, M])
        self.P_weight = P_weight
        if bias and P_store_bias is None:
            P_store_bias = derived_partition(P_weight, [slice(0, E), slice(0, 1), slice(0, 1)], [E, 1, 1])
        if bias and P_apply_bias is None:
            P_apply_bias = derived_partition(P_weight, [slice(0, E), slice(0, N), slice(0, 1)], [E, N, 1])
        self.P_store_bias, self.P_apply_bias = (P_store_bias, P_apply_bias) if bias else (None, None)
        self.e_local = int(compute_subshape(E, P_weight.index[0], [num_experts])[0])
        out_local = int(compute_subshape(N, P_weight.index[1], [out_features])[0])
        self.in_local = int(compute_subshape(M, P_weight.index[2], [in_features])[0])
        self.weight = torch.nn.Parameter(torch.empty(self.e_local, out_local, self.in_local, **kw))
        if bias and self.P_store_bias.active:
            self.bias = torch.nn.Parameter(torch.empty(self.e_local, 1, out_features, **kw))
        elif bias and self.P_apply_bias.active:
            self.register_buffer("bias", zero_volume_tensor(device=device, dtype=dtype, requires_grad=True))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        self.all_gather_weight = AllGather(P_weight, axes_all_gather=(1,), scale_backward=scale_backward)
        self.reduce_scatter_weight = ReduceScatter(P_weight, axes_reduce_scatter=(1,))
        if bias and self.P_apply_bias.active:
            self.broadcast_bias = Broadcast(self.P_store_bias, self.P_apply_bias, scale_backward=scale_backward,
                                            preserve_batch=False)
        if P_expert_seq is not None:
            self.reduce_scatter = ReduceScatter(P_expert_seq, axes_reduce_scatter=(2,))
        else:
            self.reduce_scatter = ReduceScatter(P_expert_emb, axes_reduce_scatter=(3,))
        self.prefetch = PrefetchStream(device)
        self.weight_buffer = None
        self.bias_buffer = None
        self._register_state_dict_hook(self.gather_state_dict)
        self._register_load_state_dict_pre_hook(self.scatter_state_dict)
        if collect_state:
            self.P_root = root_partition(P_weight)
            self.gather_weight = Repartition(P_weight, self.P_root, preserve_batch=False)
            self.scatter_weight = Repartition(self.P_root, P_weight, preserve_batch=False)
            if bias:
                self.gather_bias = Repartition(self.P_store_bias, self.P_root, preserve_batch=False)
                self.scatter_bias = Repartition(self.P_root, self.P_store_bias, preserve_batch=False)

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (getattr(self, "collect_state", False) and self.P_expert_emb.active):
            return destination
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        has_bias_entry = self.use_bias and bias_key in destination
        if has_bias_entry:
            bias = destination.pop(bias_key).detach()
        if self.use_bias and (self.P_store_bias.active or self.P_root.active):
            bias = self.gather_bias(bias)
        weight = self.gather_weight(destination.pop(weight_key).detach())
        if self.P_root.active:
            destination[weight_key] = weight
            if self.use_bias:
                destination[bias_key] = bias
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (getattr(self, "collect_state", False) and self.P_expert_emb.active):
            return destination
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        dev = self.P_weight.device
        weight = destination.pop(weight_key, None)
        weight = weight.to(dev) if self.P_root.active else zero_volume_tensor(device=dev, dtype=self.weight.dtype)
        destination[weight_key] = self.scatter_weight(weight)
        if self.use_bias:
            bias = destination.pop(bias_key, None)
            bias = bias.to(dev) if self.P_root.active else zero_volume_tensor(device=dev, dtype=self.weight.dtype)
            if self.P_store_bias.active or self.P_root.active:
                bias = self.scatter_bias(bias)
            if self.P_store_bias.active:
                destination[bias_key] = bias
            elif self.P_apply_bias.active:
                destination[bias_key] = zero_volume_tensor(device=dev, dtype=self.weight.dtype)
        return destination

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"num_experts={self.num_experts}, bias={self.use_bias}")

    def reset_parameters(self):
        bound = 1 / math.sqrt(self.in_features) if self.in_features > 0 else 0
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)
            if self.use_bias and self.P_store_bias.active:
                self.bias.uniform_(-bound, bound)

    def _collect_weights(self):
        w = self.all_gather_weight(self.weight)                 # [e, out, in/M]
        self.weight_buffer = w if self.auto_clear_buffer else w.detach().requires_grad_(True)
        if self.use_bias and self.P_apply_bias.active:
            self.bias_buffer = self.broadcast_bias(self.bias)

    def collect_weights(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if self.weight_buffer is None:
            self.prefetch.run(self._collect_weights)

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
            if self.scale_backward is not None:
                g = g / self.scale_backward
            gl = self.reduce_scatter_weight(g)
            deliver_grad(self.weight, gl)
        self.weight_buffer = None
        self.bias_buffer = None

    def forward(self, input):
        if not self.P_expert_emb.active:
            return input
        self.collect_weights()
        self.wait_for_streams()
        w, b = self.weight_buffer, self.bias_buffer
        e, c, s, m = input.shape
        y = _expert_matmul(input.reshape(e, c * s, m), w)
        if b is not None:
            y = y + b.reshape(e, 1, -1)
        if self.auto_clear_buffer:
            self.clear_weight_buffer()
        return self.reduce_scatter(y.reshape(e, c, s, -1))
