"""Collective part of the decomposition arithmetic
(``src/distdl/backends/common/tensor_decomposition.py:4-53``)."""
from __future__ import annotations

import numpy as np

from ...utilities.slicing import range_index
from .tensor_comm import _gather_shapes


def compute_subtensor_shapes_unbalanced(local_tensor_structure, P_in, P_out=None):
    """Table of shape ``P_in.shape + [ndim]`` with every worker's actual local
    shape, known on ``P_in`` and on ``P_out``; ``None`` elsewhere."""
    if not (P_in.active or (P_out is not None and P_out.active)):
        return None
    recs = _gather_shapes(local_tensor_structure, P_in, P_out)
    shape = [int(s) for s in P_in.shape]
    ndim = len(recs[P_in.ranks[0]][0])
    if ndim != len(shape):
        raise ValueError("tensor rank and partition rank differ")
    table = np.zeros(shape + [ndim], dtype=int)
    for flat, idx in enumerate(range_index(shape)):
        table[idx] = recs[P_in.ranks[flat]][0]
    return table
