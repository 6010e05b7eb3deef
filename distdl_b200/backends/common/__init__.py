"""Backend-independent runtime: partitions, structure exchange, buffers."""
from . import buffer, buffer_allocator, compare, convert, tensor_comm, tensor_decomposition, transport, world  # noqa: F401
from .buffer import BufferManager, ExpandableBuffer  # noqa: F401
from .partition import CartesianPartition, MPICartesianPartition, MPIPartition, Partition  # noqa: F401
from .tensor_comm import (assemble_global_tensor_structure,  # noqa: F401
                          assemble_global_tensor_structure_along_axis, broadcast_tensor_structure)
