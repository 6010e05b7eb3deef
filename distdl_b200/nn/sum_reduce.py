"""SumReduce primitive module (``src/distdl/nn/sum_reduce.py:5-192``)."""
from ..utilities.torch import TensorStructure
from .module import Module


class SumReduce(Module):
    r"""Adds the tensors of the large partition ``P_x`` onto the smaller ``P_y``
    (the mirror image of :class:`Broadcast`, whose rules apply with the roles
    swapped).  The adjoint broadcasts gradients back."""

    def __init__(self, P_x, P_y, transpose_src=False, transpose_dest=False, preserve_batch=True):
        super().__init__()
        self.P_x, self.P_y = P_x, P_y
        self.transpose_src, self.transpose_dest = transpose_src, transpose_dest
        self.preserve_batch = preserve_batch
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
            self.P_send, self.P_recv = self.P_x.create_reduction_partition_to(
                self.P_y, self.transpose_src, self.transpose_dest, initialize_backend_comm=True)
            self.input_tensor_structure = TensorStructure(input[0])
            # the structure travels from the contributors to the root: the
            # root (rank 0 of its team) needs the shape of what is reduced.
            self.output_tensor_structure = self._exchange_structure()
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])

    def _exchange_structure(self):
        """Every team agrees on the structure of the reduced tensor: it is the
        structure of any contributor's input (team rank 1 when the root itself
        does not contribute)."""
        from ..backends.common.transport import control_transport
        from ..backends.common.tensor_comm import _pack, _unpack
        ct = control_transport()
        out = self.input_tensor_structure
        teams = []
        if self.P_recv.active:
            teams.append(("root", self.P_recv))
        if self.P_send.active and not (self.P_recv.active and self.P_send.ranks == self.P_recv.ranks):
            teams.append(("member", self.P_send))
        teams.sort(key=lambda t: t[1].ranks[0])
        for role, P in teams:
            if P.size == 1:
                continue
            # source of truth: team rank 1, which always is a contributor
            payload = _pack(self.input_tensor_structure) if P.rank == 1 else None
            got = ct.broadcast_obj(payload, list(P.ranks), 1)
            if role == "root" and P.rank != 1:
                out = _unpack(got)
        return out

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
        Function = self._distdl_backend.functional.SumReduceFunction
        return Function.apply(input, self.P_send, self.P_recv, self.preserve_batch, self.input_tensor_structure,
                              self.output_tensor_structure)

    def extra_repr(self):
        return f"P_x={self.P_x.shape.tolist()}, P_y={self.P_y.shape.tolist()}"
