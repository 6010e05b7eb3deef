"""Broadcast primitive module (``src/distdl/nn/broadcast.py:7-197``)."""
from ..utilities.torch import TensorStructure
from .module import Module


class Broadcast(Module):
    r"""Copies the tensors of partition ``P_x`` onto partition ``P_y`` under the
    broadcast rules: ``P_x``'s shape, left-padded with ones, must equal
    ``P_y``'s shape or be 1 in every dimension; each ``P_x`` worker feeds the
    ``P_y`` workers that share its index in the matching dimensions.

    The adjoint sum-reduces gradients back.  ``transpose_src`` /
    ``transpose_dest`` reverse the respective shape first.  ``scale_backward``
    divides the incoming gradient.  When both partitions are the same and
    trivial (one worker, or equal transposes) the module is the identity.
    """

    def __init__(self, P_x, P_y, transpose_src=False, transpose_dest=False, preserve_batch=True,
                 scale_backward=None):
        super().__init__()
        self.P_x, self.P_y = P_x, P_y
        self.transpose_src, self.transpose_dest = transpose_src, transpose_dest
        self.preserve_batch = preserve_batch
        self.scale_backward = scale_backward
        self.identity = False
        self.input_tensor_structure = TensorStructure()
        self.output_tensor_structure = TensorStructure()
        self.P_send = self._distdl_backend.Partition([])
        self.P_recv = self._distdl_backend.Partition([])
        if P_x == P_y and (P_x.size == 1 or transpose_src == transpose_dest):
            self.identity = True

    def _distdl_module_setup(self, input):
        if not (self.P_x.active or self.P_y.active):
            self._distdl_is_setup = True
            return
        if not self.identity:
            self.P_send, self.P_recv = self.P_x.create_broadcast_partition_to(
                self.P_y, self.transpose_src, self.transpose_dest, initialize_backend_comm=True)
            self.input_tensor_structure = TensorStructure(input[0])
            self.output_tensor_structure = self._distdl_backend.broadcast_tensor_structure(
                self.input_tensor_structure, self.P_send, self.P_recv)
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])

    def _distdl_module_teardown(self, input):
        self.P_send = self._distdl_backend.Partition([])
        self.P_recv = self._distdl_backend.Partition([])
        self.input_tensor_structure = TensorStructure()
        self.output_tensor_structure = TensorStructure()
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if self.identity or not (self.P_x.active or self.P_y.active):
            return input
        Function = self._distdl_backend.functional.BroadcastFunction
        return Function.apply(input, self.P_send, self.P_recv, self.preserve_batch, self.input_tensor_structure,
                              self.output_tensor_structure, self.scale_backward)

    def extra_repr(self):
        return f"P_x={self.P_x.shape.tolist()}, P_y={self.P_y.shape.tolist()}"
