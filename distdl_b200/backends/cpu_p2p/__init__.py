"""CPU backend (selected by ``mpi``/``numpy``): tensors on the host, teams
talk through non-blocking point-to-point messages on a gloo process group.
It is the plumbing and adjoint-test path, the counterpart of the reference's
default ``mpi_numpy`` backend (``src/distdl/backends/mpi_numpy/__init__.py:1-15``).
CUDA tensors are accepted and staged through the host (the ``mpi``/``cupy``
combination)."""
import torch

from ..common import (BufferManager, CartesianPartition, ExpandableBuffer, Partition,  # noqa: F401
                      assemble_global_tensor_structure, assemble_global_tensor_structure_along_axis,
                      broadcast_tensor_structure, buffer_allocator, tensor_comm, tensor_decomposition)
from ..common.functional import bind_functional
from ..common.transport import P2PTransport

name = "mpi_numpy"
_transport = P2PTransport()
functional = bind_functional(_transport)


def transport():
    return _transport


def get_device(requested_device=None, rank=None):
    return torch.device("cpu") if requested_device is None else torch.device(requested_device)


def set_device(requested_device=None, rank=None):
    return get_device(requested_device, rank)


def prepare_team(ranks):
    """Nothing to prepare: point-to-point needs no sub-communicator."""
