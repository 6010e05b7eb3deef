"""HaloExchange primitive module (``src/distdl/nn/halo_exchange.py:5-151``)."""
import numpy as np

from ..backends.common.world import PROC_NULL
from ..utilities.torch import TensorStructure
from .module import Module


class HaloExchange(Module):
    r"""Fills the ghost (halo) regions of every worker's sub-tensor with the
    matching boundary (bulk) regions of its Cartesian neighbours.

    ``halo_shape[d] = (left, right)`` widths of the ghost regions already present
    in the input tensor; ``recv_buffer_shape`` / ``send_buffer_shape`` give the
    widths actually received / sent per side (they differ for strided
    kernels).  Dimensions are exchanged in order so that corners propagate.

    ``accumulate=True`` runs the exchange backwards instead: the ghost regions are sent to the
    neighbours they would have come from, ADDED to the bulk regions there and cleared here (for
    layers whose workers produce contributions to entries of their neighbours, such as a
    transposed convolution); the widths keep their meaning, so ``recv_buffer_shape`` is what
    leaves the ghost regions and ``send_buffer_shape`` what arrives on the bulk."""

    def __init__(self, P_x, halo_shape, recv_buffer_shape, send_buffer_shape, buffer_manager=None, accumulate=False):
        super().__init__()
        self.P_x = P_x
        self.accumulate = accumulate
        self.halo_shape = np.asarray(halo_shape, dtype=int)
        self.recv_buffer_shape = np.asarray(recv_buffer_shape, dtype=int)
        self.send_buffer_shape = np.asarray(send_buffer_shape, dtype=int)
        self.buffer_manager = buffer_manager or self._distdl_backend.BufferManager()
        self.neighbor_ranks = None
        self.slices = None
        self.buffers = None
        if P_x.active:
            team = P_x.neighbor_ranks(P_x.rank)
            # world ranks, so that the transport can address them directly
            self.neighbor_ranks = [tuple(PROC_NULL if r == PROC_NULL else P_x.ranks[r] for r in pair)
                                   for pair in team]

    def _assemble_slices(self, x_local_shape, recv_buffer_shape, send_buffer_shape):
        """Per dimension the nd-slices (left bulk, left ghost, right bulk, right
        ghost).  In dimension d the slabs span the full (ghost-including)
        extent of the dimensions already exchanged and the bulk extent of those
        still to come, which is what makes corner values arrive."""
        dim = len(x_local_shape)
        out = []
        for d in range(dim):
            def base():
                sl = []
                for k in range(dim):
                    if k < d:
                        sl.append(slice(0, int(x_local_shape[k])))
                    else:
                        lo = int(self.halo_shape[k][0])
                        hi = int(x_local_shape[k]) - int(self.halo_shape[k][1])
                        sl.append(slice(lo, hi))
                return sl
            n = int(x_local_shape[d])
            hl, hr = int(self.halo_shape[d][0]), int(self.halo_shape[d][1])
            rl, rr = int(recv_buffer_shape[d][0]), int(recv_buffer_shape[d][1])
            s_l, s_r = int(send_buffer_shape[d][0]), int(send_buffer_shape[d][1])
            lb, lg, rb, rg = base(), base(), base(), base()
            lb[d] = slice(hl, hl + s_l)
            lg[d] = slice(hl - rl, hl)
            rb[d] = slice(n - hr - s_r, n - hr)
            rg[d] = slice(n - hr, n - hr + rr)
            out.append((tuple(lb), tuple(lg), tuple(rb), tuple(rg)))
        return out

    def _distdl_module_setup(self, input):
        if self.P_x.active:
            x_local_shape = input[0].shape
            self.slices = self._assemble_slices(x_local_shape, self.recv_buffer_shape, self.send_buffer_shape)
            # staging views for the transports that move whole messages; the native transport packs
            # and unpacks inside its exchange kernel and needs none
            self.buffers = None
            if getattr(self._distdl_backend.transport(), "recv_into", False):
                self.buffers = self._distdl_backend.buffer_allocator.allocate_halo_exchange_buffers(
                    self.buffer_manager, self.slices, self.recv_buffer_shape, self.send_buffer_shape, input[0].dtype,
                    input[0].device)
            self.P_x.initialize_backend_comm()
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])

    def _distdl_module_teardown(self, input):
        self.slices, self.buffers = None, None
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if not self.P_x.active or self.P_x.size == 1:
            return input                               # no neighbours: nothing to exchange
        functional = self._distdl_backend.functional
        Function = functional.HaloAccumulateFunction if self.accumulate else functional.HaloExchangeFunction
        return Function.apply(input, self.P_x, self.slices, self.buffers, self.neighbor_ranks)
