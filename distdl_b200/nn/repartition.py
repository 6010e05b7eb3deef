"""Repartition primitive module (``src/distdl/nn/repartition.py:14-370``)."""
import numpy as np

from ..utilities.slicing import compute_nd_slice_shape, range_index
from ..utilities.tensor_decomposition import (compute_subtensor_intersection_slice,
                                              compute_subtensor_shapes_balanced,
                                              compute_subtensor_start_indices, compute_subtensor_stop_indices)
from ..utilities.torch import TensorStructure
from .module import Module


class Repartition(Module):
    r"""Moves a tensor from one Cartesian decomposition (``P_x``; sub-tensors may
    be unbalanced) to another (``P_y``; always balanced): a generalised
    all-to-all, scatter or gather.  Both partitions must have as many
    dimensions as the tensor.  The adjoint is the reverse repartition."""

    def __init__(self, P_x, P_y, preserve_batch=True, buffer_manager=None):
        super().__init__()
        self.P_x, self.P_y = P_x, P_y
        self.preserve_batch = preserve_batch
        self.identity = False
        self.buffer_manager = buffer_manager or self._distdl_backend.BufferManager()
        self.P_x_to_y_overlaps, self.P_y_to_x_overlaps = [], []
        self.P_x_to_y_buffers, self.P_y_to_x_buffers = None, None
        self.input_tensor_structure = TensorStructure()
        self.output_tensor_structure = TensorStructure()
        self.global_input_tensor_structure = TensorStructure()
        self.P_union = self._distdl_backend.Partition([])
        if not (P_x.active or P_y.active):
            return
        self.P_union = P_x.create_partition_union(P_y, initialize_backend_comm=True)
        self.P_x_shape = np.asarray(P_x.shape, dtype=int)
        self.P_y_shape = np.asarray(P_y.shape, dtype=int)
        if len(self.P_x_shape) != len(self.P_y_shape):
            raise ValueError("Input and output partition must be same dimension.")
        # world ranks of the workers of each partition, in partition-rank order
        self.P_x_ranks = np.asarray(P_x.ranks, dtype=int)
        self.P_y_ranks = np.asarray(P_y.ranks, dtype=int)
        if P_x == P_y:
            self.identity = True

    def _distdl_module_setup(self, input):
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])
        if not (self.P_x.active or self.P_y.active) or self.identity:
            return
        be = self._distdl_backend
        self.input_tensor_structure = TensorStructure(input[0])
        self.global_input_tensor_structure = be.assemble_global_tensor_structure(
            self.input_tensor_structure, self.P_x, self.P_union)
        g = self.global_input_tensor_structure
        tensor_dim = len(g.shape)
        if tensor_dim != len(self.P_x_shape):
            raise ValueError(f"Input partition mismatched: tensor has {tensor_dim} dims, partition "
                             f"{len(self.P_x_shape)}.")
        if tensor_dim != len(self.P_y_shape):
            raise ValueError("Output partition mismatched with tensor dimension.")
        if any(int(n) == 1 and int(p) > 1 for n, p in zip(g.shape, self.P_y_shape)):
            raise ValueError("Cannot split a tensor dimension of size 1 across several workers.")
        x_shapes = be.tensor_decomposition.compute_subtensor_shapes_unbalanced(
            self.input_tensor_structure, self.P_x, self.P_union)
        y_shapes = compute_subtensor_shapes_balanced(g, self.P_y_shape)
        x_lo, x_hi = compute_subtensor_start_indices(x_shapes), compute_subtensor_stop_indices(x_shapes)
        y_lo, y_hi = compute_subtensor_start_indices(y_shapes), compute_subtensor_stop_indices(y_shapes)
        self.P_x_to_y_overlaps, self.P_y_to_x_overlaps = [], []
        me_x = tuple(int(i) for i in self.P_x.index) if self.P_x.active else None
        me_y = tuple(int(i) for i in self.P_y.index) if self.P_y.active else None
        if self.P_x.active:
            for rank, iy in enumerate(range_index(self.P_y_shape)):
                sl = compute_subtensor_intersection_slice(x_lo[me_x], x_hi[me_x], y_lo[iy], y_hi[iy])
                if sl is None:
                    self.P_x_to_y_overlaps.append((None, None, None))
                    continue
                partner = int(self.P_y_ranks[rank])
                if self.P_y.active and partner == int(self.P_y_ranks[self.P_y.rank]):
                    partner = "self"
                self.P_x_to_y_overlaps.append((sl, compute_nd_slice_shape(sl), partner))
        if self.P_y.active:
            for rank, ix in enumerate(range_index(self.P_x_shape)):
                sl = compute_subtensor_intersection_slice(y_lo[me_y], y_hi[me_y], x_lo[ix], x_hi[ix])
                if sl is None:
                    self.P_y_to_x_overlaps.append((None, None, None))
                    continue
                partner = int(self.P_x_ranks[rank])
                if self.P_x.active and partner == int(self.P_x_ranks[self.P_x.rank]):
                    partner = "self"
                self.P_y_to_x_overlaps.append((sl, compute_nd_slice_shape(sl), partner))
            out = TensorStructure()
            out.shape = tuple(int(s) for s in y_shapes[me_y])
            out.dtype, out.requires_grad = g.dtype, g.requires_grad
            self.output_tensor_structure = out
        # staging views for the transports that move whole messages (the native transport needs none)
        self.P_x_to_y_buffers, self.P_y_to_x_buffers = None, None
        if getattr(be.transport(), "recv_into", False):
            self.P_x_to_y_buffers, self.P_y_to_x_buffers = be.buffer_allocator.allocate_repartition_buffers(
                self.buffer_manager, self.P_x_to_y_overlaps, self.P_y_to_x_overlaps, g.dtype, input[0].device)

    def _distdl_module_teardown(self, input):
        self.P_x_to_y_overlaps, self.P_y_to_x_overlaps = [], []
        self.P_x_to_y_buffers, self.P_y_to_x_buffers = None, None
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if not (self.P_x.active or self.P_y.active):
            return input
        if self.identity:
            return input.clone()
        Function = self._distdl_backend.functional.RepartitionFunction
        return Function.apply(input, self.P_union, self.global_input_tensor_structure, self.input_tensor_structure,
                              self.output_tensor_structure, self.P_x, self.P_x_to_y_overlaps,
                              self.P_x_to_y_buffers, self.P_y, self.P_y_to_x_overlaps, self.P_y_to_x_buffers,
                              self.preserve_batch)

    def extra_repr(self):
        return f"P_x={self.P_x.shape.tolist()}, P_y={self.P_y.shape.tolist()}"
