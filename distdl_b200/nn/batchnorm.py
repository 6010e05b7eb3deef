"""Batch normalisation over partitioned tensors (``src/distdl/nn/batchnorm.py:16-360``)."""
import numpy as np
import torch

from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import derived_partition, root_partition
from .broadcast import Broadcast
from .module import Module
from .repartition import Repartition
from .sum_reduce import SumReduce


class DistributedBatchNorm(Module):
    r"""Batch norm of ``[batch, feature, *rest]`` tensors on any Cartesian
    partition ``P_x`` (the feature dimension may be split too).  Per-feature
    sums are reduced onto ``P_sum = [1, F, 1, ...]`` (one worker per feature
    shard), turned into mean / variance there, and broadcast back; running
    statistics and the affine ``gamma`` / ``beta`` live on ``P_sum``.

    ``collect_state=True``: ``state_dict()`` holds ``gamma``, ``beta`` and the running statistics of
    ALL features, shape ``[1, F, 1, ...]``, on the first worker only, and ``load_state_dict`` takes
    them there (``src/distdl/nn/batchnorm.py:136-190``).  ``prefetch_weights()`` broadcasts
    ``gamma`` / ``beta`` ahead of the next forward (``:290-304``)."""

    def __init__(self, P_x, num_features, eps=1e-05, momentum=0.1, affine=True, track_running_stats=True,
                 device=None, dtype=None, collect_state=False, scale_backward=None):
        super().__init__()
        self.P_x = P_x
        if not P_x.active:
            return
        self.num_features, self.eps, self.momentum = num_features, eps, momentum
        self.affine, self.track_running_stats = affine, track_running_stats
        self.collect_state = collect_state
        device = device if device is not None else P_x.device
        kw = {"device": device, "dtype": dtype}
        dim, Fp = P_x.dim, int(P_x.shape[1])
        idx = [slice(0, 1)] * dim
        idx[1] = slice(0, Fp)
        shape = [1] * dim
        shape[1] = Fp
        self.P_sum = derived_partition(P_x, idx, shape)
        self.sr = SumReduce(P_x, self.P_sum, preserve_batch=False)
        self.bc = Broadcast(self.P_sum, P_x, preserve_batch=False, scale_backward=scale_backward)
        self.sr2 = SumReduce(P_x, self.P_sum, preserve_batch=False)
        self.bc2 = Broadcast(self.P_sum, P_x, preserve_batch=False, scale_backward=scale_backward)
        self.bc_g = Broadcast(self.P_sum, P_x, preserve_batch=False, scale_backward=scale_backward)
        self.bc_b = Broadcast(self.P_sum, P_x, preserve_batch=False, scale_backward=scale_backward)
        self.bc_rm = Broadcast(self.P_sum, P_x, preserve_batch=False)
        self.bc_rv = Broadcast(self.P_sum, P_x, preserve_batch=False)
        self.local_features = int(compute_subshape(Fp, P_x.index[1], [num_features])[0])
        pshape = [1] * dim
        pshape[1] = self.local_features
        self.pshape = pshape
        if self.P_sum.active:
            if affine:
                self.gamma = torch.nn.Parameter(torch.ones(pshape, **kw))
                self.beta = torch.nn.Parameter(torch.zeros(pshape, **kw))
            if track_running_stats:
                self.register_buffer("running_mean", torch.zeros(pshape, **kw))
                self.register_buffer("running_var", torch.ones(pshape, **kw))
        else:
            if affine:
                self.register_buffer("gamma", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
                self.register_buffer("beta", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
            if track_running_stats:
                self.register_buffer("running_mean", zero_volume_tensor(device=device, dtype=dtype))
                self.register_buffer("running_var", zero_volume_tensor(device=device, dtype=dtype))
        self.global_count = None
        self.gamma_buffer = self.beta_buffer = None
        self._register_state_dict_hook(self.gather_state_dict)
        self._register_load_state_dict_pre_hook(self.scatter_state_dict)
        if collect_state:
            self.P_root = root_partition(P_x)
            self.gather_affine = Repartition(self.P_sum, self.P_root, preserve_batch=False)
            self.scatter_affine = Repartition(self.P_root, self.P_sum, preserve_batch=False)

    def extra_repr(self):
        return f"num_features={self.num_features}"

    def _state_names(self):
        names = ["gamma", "beta"] if self.affine else []
        return names + (["running_mean", "running_var"] if self.track_running_stats else [])

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (getattr(self, "collect_state", False) and self.P_x.active):
            return destination
        for name in self._state_names():
            t = destination.pop(prefix + name).detach()
            if self.P_sum.active:                     # the first worker is a member of P_sum
                t = self.gather_affine(t)
            if self.P_root.active:
                destination[prefix + name] = t
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (getattr(self, "collect_state", False) and self.P_x.active):
            return destination
        dev = self.P_x.device
        for name in self._state_names():
            t = destination.pop(prefix + name, None)
            dtype = getattr(self, name).dtype
            t = t.to(dev) if self.P_root.active else zero_volume_tensor(device=dev, dtype=dtype)
            if self.P_sum.active:
                t = self.scatter_affine(t)
            destination[prefix + name] = t
        return destination

    def prefetch_weights(self):
        if self.affine and self.P_x.active:
            self.gamma_buffer = self.bc_g(self.gamma)
            self.beta_buffer = self.bc_b(self.beta)

    def _distdl_module_setup(self, input):
        self._distdl_is_setup = True
        if not self.P_x.active:
            return
        x = input[0]
        local = float(np.prod(x.shape) / x.shape[1])
        # count of entries per feature: sum over the workers sharing a feature shard
        counts = self.P_x.allgather_data(np.array([local, float(self.P_x.index[1])]))
        mine = float(self.P_x.index[1])
        self.global_count = float(sum(c[0] for c in counts if c[1] == mine))

    def forward(self, input):
        if not self.P_x.active:
            return input
        from ..ops import batchnorm as bn_ops
        if self.training or not self.track_running_stats:
            # local per-feature sums: one reduction kernel each (fp32 accumulation)
            s = self.sr(bn_ops.channel_sum(input))
            mean_root = s / self.global_count if self.P_sum.active else s
            mean = self.bc(mean_root)
            v = self.sr2(bn_ops.channel_sqdev(input, mean))
            var_root = v / self.global_count if self.P_sum.active else v
            var = self.bc2(var_root)
            if self.track_running_stats and self.P_sum.active and self.training:
                with torch.no_grad():
                    n = self.global_count
                    unbiased = var_root * (n / max(n - 1.0, 1.0))
                    self.running_mean.mul_(1 - self.momentum).add_(self.momentum * mean_root.detach())
                    self.running_var.mul_(1 - self.momentum).add_(self.momentum * unbiased.detach())
        else:
            mean = self.bc_rm(self.running_mean)
            var = self.bc_rv(self.running_var)
        gamma = beta = None
        if self.affine:
            if self.gamma_buffer is None:
                self.prefetch_weights()
            gamma, beta = self.gamma_buffer, self.beta_buffer
            self.gamma_buffer = self.beta_buffer = None
        # normalisation and affine map in one element-wise kernel (and one reduction + one element-wise
        # kernel in its backward pass)
        return bn_ops.normalize(input, mean, var, gamma, beta, self.eps)
