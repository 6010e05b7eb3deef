"""Native B200 backend (``native``/``cupy``): hand-written sm_100a kernels move
the data through peer-mapped (symmetric) memory over NVLink / NVSwitch; NCCL
carries what no kernel covers.  See :mod:`distdl_b200.parallel.symm` for the
symmetric heap and :mod:`distdl_b200.parallel.collectives` for the kernels."""
import torch

from ..common import (BufferManager, CartesianPartition, ExpandableBuffer, Partition,  # noqa: F401
                      assemble_global_tensor_structure, assemble_global_tensor_structure_along_axis,
                      broadcast_tensor_structure, buffer_allocator, tensor_comm, tensor_decomposition)
from ..common.functional import bind_functional
from ..nccl_group import get_device, set_device  # noqa: F401
from .transport import NativeTransport

name = "native_cupy"
_transport = NativeTransport()
functional = bind_functional(_transport)


def transport():
    return _transport


def prepare_team(ranks):
    _transport.prepare(ranks)
