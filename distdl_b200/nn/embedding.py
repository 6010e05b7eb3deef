"""Embedding with the table split over its embedding dimension
(``src/distdl/nn/embedding.py:14-246``)."""
import torch

from .. import ops
from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import derived_partition
from .broadcast import Broadcast
from .module import Module
from .repartition import Repartition


class DistributedEmbedding(Module):
    r"""Look-up table ``[num_embeddings, embedding_dim]`` whose columns are split
    over the last dimension of ``P_x = [D, ..., M]``: each worker returns its
    ``embedding_dim / M`` slice of every looked-up row.  The table shard lives
    on the first data-parallel row (``P_weight = [1, ..., M]``) and is broadcast
    to the others.  The full table is drawn on the root and scattered, so the
    initial values do not depend on the number of workers.  A sequence-sharded
    input is not supported (as in the reference)."""

    def __init__(self, P_x, num_embeddings, embedding_dim, padding_idx=None, max_norm=None, norm_type=2.,
                 scale_grad_by_freq=False, sparse=False, _weight=None, _freeze=False, collect_state=False,
                 device=None, dtype=None, scale_backward=None):
        super().__init__()
        self.P_x = P_x
        if not P_x.active:
            return
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.padding_idx, self.max_norm, self.norm_type = padding_idx, max_norm, norm_type
        self.scale_grad_by_freq, self.sparse = scale_grad_by_freq, sparse
        self.collect_state, self.dtype = collect_state, dtype
        device = device if device is not None else P_x.device
        self._device = device
        dim, M = P_x.dim, int(P_x.shape[-1])
        idx = [slice(0, 1)] * dim
        idx[-1] = slice(0, M)
        self.P_weight = derived_partition(P_x, idx, [1, M])
        # same workers seen as a [1, ..., M] grid of P_x's rank for the broadcast rules
        self.P_weight_bcast = derived_partition(P_x, idx, [1] * (dim - 1) + [M])
        self.broadcast_weight = Broadcast(self.P_weight_bcast, P_x, scale_backward=scale_backward)
        self.P_root = P_x.create_partition_inclusive([0]).create_cartesian_topology_partition([1, 1])
        self.scatter_weight = Repartition(self.P_root, self.P_weight, preserve_batch=False)
        self.gather_weight = Repartition(self.P_weight, self.P_root, preserve_batch=False)
        if self.P_weight.active:
            local = int(compute_subshape(M, self.P_weight.index[-1], [embedding_dim])[0])
            self.weight = torch.nn.Parameter(torch.empty(num_embeddings, local, device=device, dtype=dtype),
                                             requires_grad=not _freeze)
        else:
            self.register_buffer("weight", zero_volume_tensor(device=device, requires_grad=True, dtype=dtype))
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
        if self.P_weight.active or self.P_root.active:
            with torch.no_grad():
                shard = self.scatter_weight(full)
                if self.P_weight.active:
                    self.weight.copy_(shard)

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        key = prefix + "weight"
        w = destination.pop(key)
        if self.P_weight.active or self.P_root.active:
            full = self.gather_weight(w.detach() if self.P_weight.active else
                                      zero_volume_tensor(device=self._device, dtype=self.dtype))
            if self.P_root.active:
                destination[key] = full
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        key = prefix + "weight"
        w = destination.pop(key, None)
        if self.P_weight.active or self.P_root.active:
            full = w.to(self._device) if self.P_root.active else zero_volume_tensor(device=self._device,
                                                                                    dtype=self.dtype)
            shard = self.scatter_weight(full)
            if self.P_weight.active:
                destination[key] = shard
                return destination
        destination[key] = zero_volume_tensor(device=self._device, dtype=self.dtype)
        return destination

    def extra_repr(self):
        return f"num_embeddings={self.num_embeddings}, embedding_dim={self.embedding_dim}"

    def prefetch_weights(self):
        """Broadcasts the table over the data-parallel workers ahead of the next forward
        (``src/distdl/nn/embedding.py:213-220``)."""
        if not self.P_x.active:
            return
        w = self.weight
        if self.P_weight_bcast.active:
            w = w.reshape([1] * (self.P_x.dim - 2) + list(self.weight.shape))
        self.weight_buffer = self.broadcast_weight(w).reshape(self.num_embeddings, -1)

    def forward(self, input):
        if not self.P_x.active:
            return input
        if self.weight_buffer is None:
            self.prefetch_weights()
        w, self.weight_buffer = self.weight_buffer, None
        if self.max_norm is None and not self.scale_grad_by_freq and not self.sparse:
            return ops.embedding(input, w, self.padding_idx)
        return torch.nn.functional.embedding(input, w, self.padding_idx, self.max_norm, self.norm_type,
                                             self.scale_grad_by_freq, self.sparse)
