"""Embedding with the table split over both the vocabulary (data-parallel
workers, ZeRO-3) and the embedding dimension (tensor-parallel workers)
(``src/distdl/nn/embedding_zero.py:15-278``)."""
import torch

from .. import ops
from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import KeptBufferGuard, PrefetchStream, reduce_scatter_grad
from .all_gather import AllGather
from .module import Module
from .reduce_scatter import ReduceScatter
from .repartition import Repartition


class DistributedEmbeddingZero(Module):
    r"""Table shard ``[num_embeddings / D, embedding_dim / M]`` on every worker of
    ``P_x = [D, ..., M]``.  Forward all-gathers the rows over ``D`` and looks
    up; autograd reduce-scatters the table gradient back.  ``auto_clear_buffer=False``
    keeps the gathered table across micro-batches."""

    def __init__(self, P_x, num_embeddings, embedding_dim, padding_idx=None, max_norm=None, norm_type=2.,
                 scale_grad_by_freq=False, sparse=False, _weight=None, _freeze=False, collect_state=False,
                 device=None, dtype=None, scale_backward=None, auto_clear_buffer=True):
        super().__init__()
        self.P_x = P_x
        if not P_x.active:
            return
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx, self.max_norm, self.norm_type = padding_idx, max_norm, norm_type
        self.scale_grad_by_freq, self.sparse = scale_grad_by_freq, sparse
        self.collect_state, self.dtype = collect_state, dtype
        self.scale_backward, self.auto_clear_buffer = scale_backward, auto_clear_buffer
        device = device if device is not None else P_x.device
        self._device = device
        D, M = int(P_x.shape[0]), int(P_x.shape[-1])
        # the table is 2-D: view the workers as a [D * (middle dims), M] grid
        mid = int(P_x.size // (D * M))
        if mid != 1:
            raise ValueError("DistributedEmbeddingZero expects partition shape [D, 1, ..., M]")
        self.P_weight = P_x.create_partition_inclusive(range(P_x.size)).create_cartesian_topology_partition([D, M])
        self.allgather = AllGather(self.P_weight, axes_all_gather=(0,), scale_backward=scale_backward)
        self.reduce_scatter = ReduceScatter(self.P_weight, axes_reduce_scatter=(0,))
        rows = int(compute_subshape(D, self.P_weight.index[0], [num_embeddings])[0])
        cols = int(compute_subshape(M, self.P_weight.index[1], [embedding_dim])[0])
        self.weight = torch.nn.Parameter(torch.empty(rows, cols, device=device, dtype=dtype),
                                         requires_grad=not _freeze)
        self.P_root = P_x.create_partition_inclusive([0]).create_cartesian_topology_partition([1, 1])
        self.scatter_weight = Repartition(self.P_root, self.P_weight, preserve_batch=False)
        self.gather_weight = Repartition(self.P_weight, self.P_root, preserve_batch=False)
        self.prefetch = PrefetchStream(device)
        self._kept = KeptBufferGuard()
        self.weight_buffer = None
        self.reset_parameters(_weight)
        self._register_state_dict_hook(self.gather_state_dict)
        self._register_load_state_dict_pre_hook(self.scatter_state_dict)

    def reset_parameters(self, _weight=None):
        full = zero_volume_tensor(device=self._device, dtype=self.dtype)
        if self.P_root.active:
            full = _weight.to(self._device) if _weight is not None else torch.randn(
                self.num_embeddings, self.embedding_dim, device=self._device, dtype=self.dtype)
            if self.padding_idx is not None:
                with torch.no_grad():
                    full[self.padding_idx].zero_()
        with torch.no_grad():
            self.weight.copy_(self.scatter_weight(full))

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        key = prefix + "weight"
        full = self.gather_weight(destination.pop(key).detach())
        if self.P_root.active:
            destination[key] = full
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        key = prefix + "weight"
        w = destination.pop(key, None)
        full = w.to(self._device) if self.P_root.active else zero_volume_tensor(device=self._device, dtype=self.dtype)
        destination[key] = self.scatter_weight(full)
        return destination

    def _collect(self):
        w = self.allgather(self.weight)
        self.weight_buffer = w if self.auto_clear_buffer else w.detach().requires_grad_(True)

    def collect_weights(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if self.weight_buffer is not None and not self.auto_clear_buffer and self._kept.stale(self.weight):
            self.weight_buffer = None
        if self.weight_buffer is None:
            self.prefetch.run(self._collect)
            self._kept.remember(self.weight)

    prefetch_weights = collect_weights

    def wait_for_streams(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        self.prefetch.wait()

    def clear_weight_buffer(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if not self.auto_clear_buffer and self.weight_buffer is not None and self.weight_buffer.grad is not None:
            reduce_scatter_grad(self.reduce_scatter, self.weight_buffer.grad, self.weight, self.scale_backward)
        self.weight_buffer = None

    def forward(self, input):
        if not self.P_x.active:
            return input
        self.collect_weights()
        self.wait_for_streams()
        w = self.weight_buffer
        if self.max_norm is None and not self.scale_grad_by_freq and not self.sparse:
            y = ops.embedding(input, w, self.padding_idx)
        else:
            y = torch.nn.functional.embedding(input, w, self.padding_idx, self.max_norm, self.norm_type,
                                              self.scale_grad_by_freq, self.sparse)
        if self.auto_clear_buffer:
            self.clear_weight_buffer()
        return y
