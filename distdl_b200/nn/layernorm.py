"""LayerNorm over tensors whose normalised dimensions may be partitioned
(``src/distdl/nn/layernorm.py:16-321``)."""
import numpy as np
import torch

from .. import ops
from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import derived_partition, root_partition
from .all_sum_reduce import AllSumReduce
from .broadcast import Broadcast
from .module import Module
from .repartition import Repartition


class DistributedLayerNorm(Module):
    r"""Layer normalisation over the last ``len(normalized_shape)`` dimensions.

    When those dimensions are split across workers (tensor parallelism over the
    features), the row statistics are completed with ONE all-reduce of the
    per-row ``(sum, sum of squares, count)`` triple -- exact for unequal shard
    sizes (the reference averages shard means with two all-reduces, which is
    exact only for equal shards, ``src/distdl/nn/layernorm.py:218-247``).
    When they are local (sequence parallelism) the fused LayerNorm kernel runs
    with no communication.  The affine parameters are sharded like the
    normalised dimensions on the first worker of every other dimension
    (``P_w``) and broadcast to the rest.
    """

    def __init__(self, P_x, normalized_shape, elementwise_affine=True, eps=1e-5, collect_state=False, device=None,
                 dtype=None, scale_backward=None):
        super().__init__()
        self.P_x = P_x
        if not P_x.active:
            return
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(int(s) for s in normalized_shape)
        self.elementwise_affine, self.eps, self.collect_state = elementwise_affine, eps, collect_state
        self.dtype = dtype
        device = device if device is not None else P_x.device
        kw = {"device": device, "dtype": dtype}
        dim, nn = P_x.dim, len(self.normalized_shape)
        self.dim_reduce = tuple(range(dim - nn, dim))
        self.num_reduce = int(np.prod([int(P_x.shape[d]) for d in self.dim_reduce]))
        self.allreduce = AllSumReduce(P_x, axes_reduce=self.dim_reduce)
        if elementwise_affine:
            idx = [slice(0, 1)] * dim
            shape = [1] * dim
            for d in self.dim_reduce:
                idx[d] = slice(0, int(P_x.shape[d]))
                shape[d] = int(P_x.shape[d])
            self.P_w = derived_partition(P_x, idx, shape)
            self.broadcast_weight = Broadcast(self.P_w, P_x, scale_backward=scale_backward)
            self.broadcast_bias = Broadcast(self.P_w, P_x, scale_backward=scale_backward)
            if self.P_w.active:
                gshape = [1] * (dim - nn) + list(self.normalized_shape)
                local = [int(s) for s in compute_subshape(self.P_w.shape, self.P_w.index, gshape)]
                self.weight = torch.nn.Parameter(torch.ones(tuple(local), **kw))
                self.bias = torch.nn.Parameter(torch.zeros(tuple(local), **kw))
            else:
                self.register_buffer("weight", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
                self.register_buffer("bias", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
            self._register_state_dict_hook(self.gather_state_dict)
            self._register_load_state_dict_pre_hook(self.scatter_state_dict)
            if collect_state:
                self.P_root = root_partition(P_x)
                self.gather = Repartition(self.P_w, self.P_root, preserve_batch=False)
                self.scatter = Repartition(self.P_root, self.P_w, preserve_batch=False)
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)
        self.weight_buffer = self.bias_buffer = None

    def reset_parameters(self):
        if self.elementwise_affine and self.P_w.active:
            with torch.no_grad():
                self.weight.fill_(1.0)
                self.bias.zero_()

    def extra_repr(self):
        return f"normalized_shape={self.normalized_shape}"

    def prefetch_weights(self):
        """Broadcasts the affine parameters ahead of the next forward
        (``src/distdl/nn/layernorm.py:249-263``)."""
        if self.P_x.active and self.elementwise_affine:
            self.weight_buffer = self.broadcast_weight(self.weight)
            self.bias_buffer = self.broadcast_bias(self.bias)

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active and self.elementwise_affine):
            return destination
        for name in ("bias", "weight"):
            key = prefix + name
            t = self.gather(destination.pop(key).detach())
            if self.P_root.active:
                destination[key] = t.reshape(self.normalized_shape)
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active and self.elementwise_affine):
            return destination
        dim, nn = self.P_x.dim, len(self.normalized_shape)
        for name in ("weight", "bias"):
            key = prefix + name
            t = destination.pop(key, None)
            if self.P_root.active:
                t = t.reshape([1] * (dim - nn) + list(self.normalized_shape)).to(self.P_x.device)
            else:
                t = zero_volume_tensor(device=self.P_x.device, dtype=self.dtype)
            destination[key] = self.scatter(t)
        return destination

    def forward(self, input):
        if not self.P_x.active:
            return input
        w = b = None
        if self.elementwise_affine:
            if self.weight_buffer is None:
                self.prefetch_weights()
            w, b = self.weight_buffer, self.bias_buffer
            self.weight_buffer = self.bias_buffer = None
        nn = len(self.normalized_shape)
        if self.num_reduce == 1:
            if nn == 1:
                return ops.layer_norm(input, None if w is None else w.reshape(-1), None if b is None else b.reshape(-1),
                                      self.eps)
            shape = tuple(input.shape[-nn:])
            return torch.nn.functional.layer_norm(input, shape, None if w is None else w.reshape(shape),
                                                  None if b is None else b.reshape(shape), self.eps)
        if nn == 1 and input.is_cuda and getattr(self._distdl_backend, "name", "") == "native_cupy":
            # feature-split rows on the native backend: statistics exchange fused into the norm kernel
            from ..parallel import split_norm
            team = getattr(self, "_stat_team", None)
            if team is None:
                team = tuple(self.P_x.create_allreduction_partition(self.dim_reduce).ranks)
                object.__setattr__(self, "_stat_team", team)
            if split_norm.usable(input, w, b, team):
                return split_norm.split_norm(input, w, b, self.eps, team, self.normalized_shape[0])
        dims = tuple(range(input.dim() - nn, input.dim()))
        xf = input.float()
        local_n = float(np.prod([input.shape[d] for d in dims]))
        stats = torch.stack([xf.sum(dims), (xf * xf).sum(dims), torch.full_like(xf.sum(dims), local_n)], dim=-1)
        stats = self.allreduce(stats)
        n = stats[..., 2]
        mean = stats[..., 0] / n
        var = (stats[..., 1] / n - mean * mean).clamp_min(0.0)
        for _ in dims:
            mean, var = mean.unsqueeze(-1), var.unsqueeze(-1)
        y = (xf - mean) * torch.rsqrt(var + self.eps)
        if w is not None:
            y = y * w.float() + b.float()
        return y.to(input.dtype)
