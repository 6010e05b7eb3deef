"""Pure helper functions: index arithmetic of balanced tensor decompositions,
dtype tables, zero-volume tensors, small debugging aids."""
from . import debug, dtype, index_tricks, misc, slicing, tensor_decomposition, torch  # noqa: F401
