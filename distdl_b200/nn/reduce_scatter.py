"""ReduceScatter primitive module (``src/distdl/nn/reduce_scatter.py:6-169``)."""
import torch

from ..utilities.slicing import compute_subshape_along_axis
from ..utilities.torch import TensorStructure
from .all_sum_reduce import _axes_from
from .module import Module


class ReduceScatter(Module):
    r"""Sums the (full-size) tensors of the workers that differ only in partition
    dimension ``axes_reduce_scatter[0]`` and leaves every worker with its
    balanced slice of the sum along that tensor dimension.  Adjoint: all-gather."""

    def __init__(self, P_x, axes_reduce_scatter=None, axes_keep=None):
        super().__init__()
        self.P_x = P_x
        self.identity = P_x.size == 1
        self.axes_reduce_scatter = _axes_from(P_x, axes_reduce_scatter, axes_keep, "axes_reduce_scatter")
        self.P_reducescatter = self._distdl_backend.Partition([])
        self.input_tensor_structure = TensorStructure()
        self.output_tensor_structure = TensorStructure()

    def _distdl_module_setup(self, input):
        if self.P_x.active and not self.identity:
            self.P_reducescatter = self.P_x.create_allreduction_partition(self.axes_reduce_scatter,
                                                                          initialize_backend_comm=True)
            self.input_tensor_structure = TensorStructure(input[0])
            axis = self.axes_reduce_scatter[0]
            out = TensorStructure(input[0])
            shape = compute_subshape_along_axis(self.P_reducescatter.shape, self.P_reducescatter.index,
                                                list(input[0].shape), axis)
            out.shape = torch.Size(int(s) for s in shape)
            self.output_tensor_structure = out
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])

    def _distdl_module_teardown(self, input):
        self.P_reducescatter = self._distdl_backend.Partition([])
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if self.identity or not self.P_x.active:
            return input
        if self.P_reducescatter.size == 1:
            return input
        Function = self._distdl_backend.functional.ReduceScatterFunction
        return Function.apply(input, self.P_reducescatter, self.input_tensor_structure,
                              self.output_tensor_structure, self.axes_reduce_scatter)

    def accumulate_into(self, input, acc, scale=1.0):
        """Fused form for gradients: ``acc += scale * reduce_scatter(input)`` with a
        flat fp32 accumulator of the size of this worker's slice.  Returns False
        (and does nothing) when the transport has no such kernel or the layout is
        not the equal split along dimension 0 that it serves."""
        if self.identity or not self.P_x.active or not input.is_cuda or self.axes_reduce_scatter[0] != 0:
            return False
        self._distdl_forward_pre_hook(self, (input,))
        P = self.P_reducescatter
        if P.size == 1 or input.shape[0] % P.size or acc.numel() * P.size != input.numel():
            return False
        t = self._distdl_backend.functional.ReduceScatterFunction.transport()
        if not hasattr(t, "reduce_scatter_accumulate"):
            return False
        return bool(t.reduce_scatter_accumulate(input.contiguous().reshape(P.size, -1), acc, list(P.ranks), scale))

    def extra_repr(self):
        return f"P_x={self.P_x.shape.tolist()}, axes_reduce_scatter={self.axes_reduce_scatter}"
