"""AllSumReduce primitive module (``src/distdl/nn/all_sum_reduce.py:5-164``)."""
from ..utilities.torch import TensorStructure
from .module import Module


def _axes_from(P_x, axes, axes_keep, what):
    if (axes is None) == (axes_keep is None):
        raise ValueError(f"Exactly one of {what} and axes_keep must be given.")
    if axes is None:
        keep = set(int(a) for a in axes_keep)
        return tuple(k for k in range(P_x.dim) if k not in keep)
    return tuple(int(a) for a in axes)


class AllSumReduce(Module):
    r"""Sums tensors across the workers that differ only in the partition
    dimensions ``axes_reduce`` (or in all but ``axes_keep``); every worker of
    such a group ends with the sum.  Self-adjoint.  Identity on one worker."""

    def __init__(self, P_x, axes_reduce=None, axes_keep=None, scale_backward=None):
        super().__init__()
        self.P_x = P_x
        self.scale_backward = scale_backward
        self.identity = P_x.size == 1
        self.axes_reduce = _axes_from(P_x, axes_reduce, axes_keep, "axes_reduce") if P_x.active or not self.identity \
            else ()
        self.P_allreduce = self._distdl_backend.Partition([])
        self.input_tensor_structure = TensorStructure()
        self.output_tensor_structure = TensorStructure()

    def _distdl_module_setup(self, input):
        if self.P_x.active and not self.identity:
            self.P_allreduce = self.P_x.create_allreduction_partition(self.axes_reduce,
                                                                      initialize_backend_comm=True)
            self.input_tensor_structure = TensorStructure(input[0])
            self.output_tensor_structure = self.input_tensor_structure
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])

    def _distdl_module_teardown(self, input):
        self.P_allreduce = self._distdl_backend.Partition([])
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if self.identity or not self.P_x.active:
            return input
        Function = self._distdl_backend.functional.AllSumReduceFunction
        return Function.apply(input, self.P_allreduce, self.input_tensor_structure, self.output_tensor_structure,
                              self.scale_backward)

    def extra_repr(self):
        return f"P_x={self.P_x.shape.tolist()}, axes_reduce={self.axes_reduce}"
