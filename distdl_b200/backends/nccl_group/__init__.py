"""NCCL backend (``nccl``/``cupy``): library collectives of ``torch.distributed``
on cached sub-groups, CUDA tensors.  Counterpart of the reference's
``nccl_cupy`` backend (``src/distdl/backends/nccl_cupy/nccl_comm.py:132-485``);
it is the measured baseline and the fallback of the native backend."""
import torch

from ..common import (BufferManager, CartesianPartition, ExpandableBuffer, Partition,  # noqa: F401
                      assemble_global_tensor_structure, assemble_global_tensor_structure_along_axis,
                      broadcast_tensor_structure, buffer_allocator, tensor_comm, tensor_decomposition)
from ..common.functional import bind_functional
from ..common.transport import GroupTransport

name = "nccl_cupy"
_transport = GroupTransport()
functional = bind_functional(_transport)


def transport():
    return _transport


def get_device(requested_device=None, rank=None):
    if requested_device is not None:
        return torch.device(requested_device)
    if not torch.cuda.is_available():
        return torch.device("cpu")
    if rank is None:
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cuda", int(rank) % torch.cuda.device_count())


def set_device(requested_device=None, rank=None):
    dev = get_device(requested_device, rank)
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    return dev


def prepare_team(ranks):
    """Creates (or fetches) the NCCL sub-group of a team; members only."""
    import torch.distributed as dist
    if dist.is_initialized() and len(ranks) > 1:
        _transport.subgroup(ranks)
