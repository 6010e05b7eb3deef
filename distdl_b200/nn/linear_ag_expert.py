"""Expert-parallel column-parallel linear layer
(``src/distdl/nn/linear_ag_expert.py:22-422``)."""
import math

import torch

from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import PrefetchStream, deliver_grad, derived_partition, relayout, root_partition, var_blocks
from .all_gather import AllGather
from .broadcast import Broadcast
from .module import Module
from .reduce_scatter import ReduceScatter
from .repartition import Repartition


def _expert_matmul(x, w):
    """x [e, rows, in], w [e, out, in] -> [e, rows, out] (grouped GEMM on the native kernel on CUDA)."""
    from ..models.moe import batched_linear
    return batched_linear(x, w)


class DistributedExpertAllGather(Module):
    r"""One linear map per expert, ``y[e] = x[e] W[e]^T + b[e]``, on routed tokens
    ``[expert, capacity, seq, feat]``.

    ``P_expert_emb = [E, N, 1, M]``: experts split over ``E`` (expert
    parallelism), capacity over ``N`` (data parallelism inside an expert
    group), features over ``M`` (tensor parallelism); ``P_expert_seq =
    [E, N, S, 1]`` selects sequence-sharded input instead.  Weight shard
    ``[experts/E, in/N, out/M]`` on ``P_weight = [E, N, M]``: ZeRO-sharded over
    ``N`` along the input features, gathered on use; bias ``[experts/E, 1,
    out/M]`` on the first ``N`` row.  Forward: gather weight, broadcast bias,
    all-gather the tokens over ``M`` (features, or sequence), grouped GEMM.
    ``auto_clear_buffer=False`` keeps the gathered weights across micro-batches.

    ``collect_state=True``: ``state_dict()`` holds, on the first worker only, the whole weight
    ``[experts, in, out]`` and bias ``[experts, 1, out]`` (with ``geglu=True`` the two halves of
    the output features in the order a single worker would store them); ``load_state_dict``
    takes that layout on the first worker and scatters it
    (``src/distdl/nn/linear_ag_expert.py:247-323``)."""

    def __init__(self, P_expert_emb, num_experts, in_features, out_features, bias=True, device=None, dtype=None,
                 P_weight=None, P_bias=None, collect_state=False, scale_backward=None, P_expert_seq=None,
                 auto_clear_buffer=True, geglu=False):
        super().__init__()
        self.P_expert_emb, self.P_expert_seq = P_expert_emb, P_expert_seq
        if not P_expert_emb.active:
            return
        assert P_expert_emb.dim == 4
        device = device if device is not None else P_expert_emb.device
        kw = {"device": device, "dtype": dtype}
        self.num_experts, self.in_features, self.out_features = num_experts, in_features, out_features
        self.use_bias, self.geglu, self.collect_state = bias, geglu, collect_state
        self.scale_backward, self.auto_clear_buffer, self.dtype = scale_backward, auto_clear_buffer, dtype
        E, N, M = (int(P_expert_emb.shape[i]) for i in (0, 1, 3))
        if P_weight is None:
            P_weight = P_expert_emb.create_partition_inclusive(range(P_expert_emb.size)) \
                .create_cartesian_topology_partition([E, N, M])
        self.P_weight = P_weight
        if bias and P_bias is None:
            P_bias = derived_partition(P_weight, [slice(0, E), slice(0, 1), slice(0, M)], [E, 1, M])
        self.P_bias = P_bias if bias else None
        self.e_local = int(compute_subshape(E, P_weight.index[0], [num_experts])[0])
        in_local = int(compute_subshape(N, P_weight.index[1], [in_features])[0])
        self.out_local = int(compute_subshape(M, P_weight.index[2], [out_features])[0])
        self.weight = torch.nn.Parameter(torch.empty(self.e_local, in_local, self.out_local, **kw))
        if bias and self.P_bias.active:
            self.bias = torch.nn.Parameter(torch.empty(self.e_local, 1, self.out_local, **kw))
        elif bias:
            self.register_buffer("bias", zero_volume_tensor(device=device, dtype=dtype, requires_grad=True))
        else:
            self.register_parameter("bias", None)
        self.reset_parameters()
        if P_expert_seq is not None:
            self.all_gather_hidden = AllGather(P_expert_seq, axes_all_gather=(2,))
        else:
            self.all_gather_hidden = AllGather(P_expert_emb, axes_all_gather=(3,))
        self.all_gather_weight = AllGather(P_weight, axes_all_gather=(1,), scale_backward=scale_backward)
        self.reduce_scatter_weight = ReduceScatter(P_weight, axes_reduce_scatter=(1,))
        if bias:
            self.broadcast_bias = Broadcast(self.P_bias, P_weight, scale_backward=scale_backward,
                                            preserve_batch=False)
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
                self.gather_bias = Repartition(self.P_bias, self.P_root, preserve_batch=False)
                self.scatter_bias = Repartition(self.P_root, self.P_bias, preserve_batch=False)

    def _geglu_blocks(self):
        return var_blocks(self.out_features, int(self.P_weight.shape[-1]), geglu=True) if self.geglu else None

    def geglu_weight_to_serial(self, weight):
        """Output features from the per-worker order ``(worker, half)`` to the serial ``(half, worker)``."""
        return relayout(weight, -1, self._geglu_blocks(), to_serial=True)

    def geglu_weight_to_parallel(self, weight):
        return relayout(weight, -1, self._geglu_blocks(), to_serial=False)

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (getattr(self, "collect_state", False) and self.P_expert_emb.active):
            return destination
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        if self.use_bias:
            bias = destination.pop(bias_key).detach()
            if self.P_bias.active or self.P_root.active:
                bias = self.gather_bias(bias)
        weight = self.gather_weight(destination.pop(weight_key).detach())
        if self.P_root.active:
            destination[weight_key] = self.geglu_weight_to_serial(weight)
            if self.use_bias:
                destination[bias_key] = self.geglu_weight_to_serial(bias)
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (getattr(self, "collect_state", False) and self.P_expert_emb.active):
            return destination
        weight_key, bias_key = prefix + "weight", prefix + "bias"
        dev = self.P_weight.device
        weight = destination.pop(weight_key, None)
        if self.P_root.active:
            weight = self.geglu_weight_to_parallel(weight.to(dev))
        else:
            weight = zero_volume_tensor(device=dev, dtype=self.weight.dtype)
        destination[weight_key] = self.scatter_weight(weight)
        if self.use_bias:
            bias = destination.pop(bias_key, None)
            if self.P_root.active:
                bias = self.geglu_weight_to_parallel(bias.to(dev))
            else:
                bias = zero_volume_tensor(device=dev, dtype=self.weight.dtype)
            if self.P_bias.active or self.P_root.active:
                bias = self.scatter_bias(bias)
            destination[bias_key] = bias if self.P_bias.active else zero_volume_tensor(device=dev,
                                                                                     dtype=self.weight.dtype)
        return destination

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, "
                f"num_experts={self.num_experts}, bias={self.use_bias}")

    def reset_parameters(self):
        bound = 1 / math.sqrt(self.in_features) if self.in_features > 0 else 0
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)
            if self.use_bias and self.P_bias.active:
                self.bias.uniform_(-bound, bound)

    def _collect_weights(self):
        w = self.all_gather_weight(self.weight)                 # [e, in, out/M]
        self.weight_buffer = w if self.auto_clear_buffer else w.detach().requires_grad_(True)
        if self.use_bias:
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
        x = self.all_gather_hidden(input)                       # [e, c, s, in]
        e, c, s, m = x.shape
        y = _expert_matmul(x.reshape(e, c * s, m), w.transpose(1, 2))
        if b is not None:
            y = y + b.reshape(e, 1, -1)
        if self.auto_clear_buffer:
            self.clear_weight_buffer()
        return y.reshape(e, c, s, -1)
