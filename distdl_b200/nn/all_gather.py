"""AllGather primitive module (``src/distdl/nn/all_gather.py:5-173``)."""
from ..utilities.torch import TensorStructure
from .all_sum_reduce import _axes_from
from .module import Module


class AllGather(Module):
    r"""Concatenates, along tensor dimension ``axes_all_gather[0]``, the shards
    held by the workers that differ only in that partition dimension; every
    worker of the group ends with the concatenation.  Adjoint: reduce-scatter."""

    def __init__(self, P_x, axes_all_gather=None, axes_keep=None, scale_backward=None):
        super().__init__()
        self.P_x = P_x
        self.scale_backward = scale_backward
        self.identity = P_x.size == 1
        self.axes_all_gather = _axes_from(P_x, axes_all_gather, axes_keep, "axes_all_gather")
        self.P_allgather = self._distdl_backend.Partition([])
        self.input_tensor_structure = TensorStructure()
        self.output_tensor_structure = TensorStructure()

    def _distdl_module_setup(self, input):
        if self.P_x.active and not self.identity:
            self.P_allgather = self.P_x.create_allreduction_partition(self.axes_all_gather,
                                                                      initialize_backend_comm=True)
            self.input_tensor_structure = TensorStructure(input[0])
            self.output_tensor_structure = self._distdl_backend.assemble_global_tensor_structure_along_axis(
                self.input_tensor_structure, self.P_allgather, self.axes_all_gather[0])
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])

    def _distdl_module_teardown(self, input):
        self.P_allgather = self._distdl_backend.Partition([])
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if self.identity or not self.P_x.active:
            return input
        if self.P_allgather.size == 1:
            return input
        Function = self._distdl_backend.functional.AllGatherFunction
        return Function.apply(input, self.P_allgather, self.input_tensor_structure, self.output_tensor_structure,
                              self.axes_all_gather, self.scale_backward)

    def extra_repr(self):
        return f"P_x={self.P_x.shape.tolist()}, axes_all_gather={self.axes_all_gather}"
