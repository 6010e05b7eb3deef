"""Tables of sub-tensor shapes / start / stop indices for every worker of a
partition (local computation only; the collective variant for unbalanced
inputs lives in ``backends.common.tensor_decomposition``).
Reference: ``src/distdl/utilities/tensor_decomposition.py:8-190``."""
from __future__ import annotations

import numpy as np

from .slicing import assemble_slices, compute_intersection, compute_subshape, range_index


def compute_subtensor_shapes_balanced(global_tensor_structure, P_tensor_shape):
    """Array of shape ``P_tensor_shape + [ndim]`` holding every worker's balanced sub-tensor shape."""
    gshape = np.asarray(global_tensor_structure.shape, dtype=int)
    P_shape = [int(p) for p in P_tensor_shape]
    if len(P_shape) != len(gshape):
        raise ValueError("tensor rank and partition rank differ")
    out = np.zeros(P_shape + [len(gshape)], dtype=int)
    for idx in range_index(P_shape):
        out[idx] = compute_subshape(P_shape, idx, gshape)
    return out


def compute_subtensor_start_indices(shapes):
    """Start indices from a table of (possibly unbalanced) shapes: along each
    dimension the start is the sum of the extents of the preceding workers."""
    shapes = np.asarray(shapes, dtype=int)
    ndim = shapes.shape[-1]
    starts = np.zeros_like(shapes)
    for d in range(ndim):
        # extents along dim d, as a function of the worker coordinate in dim d
        ext = shapes[..., d]
        csum = np.cumsum(ext, axis=d) - ext
        starts[..., d] = csum
    return starts


def compute_subtensor_stop_indices(shapes):
    shapes = np.asarray(shapes, dtype=int)
    return compute_subtensor_start_indices(shapes) + shapes


def compute_subtensor_intersection_slice(x_start_index, x_stop_index, y_start_index, y_stop_index):
    """Slices relative to x of the overlap of boxes x and y, or ``None``."""
    lo, _, extent = compute_intersection(x_start_index, x_stop_index, y_start_index, y_stop_index)
    if int(np.prod(extent)) == 0:
        return None
    rel = lo - np.asarray(x_start_index, dtype=int)
    return assemble_slices(rel, rel + extent)
