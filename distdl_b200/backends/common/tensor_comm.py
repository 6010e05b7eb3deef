"""Exchange of tensor *structure* (shape, dtype, requires_grad) between workers.

Counterpart of ``src/distdl/backends/common/tensor_comm.py:11-188``.  The
reference issues four non-blocking MPI all-reduces per side and one
communicator split per tensor dimension; because partitions here are plain
rank lists, each function is a single small message round on the control
plane (or no message at all when one worker is involved).
"""
from __future__ import annotations

import numpy as np
import torch

from ...utilities.dtype import id_to_torch_dtype, torch_dtype_to_id
from ...utilities.slicing import range_index
from ...utilities.torch import TensorStructure
from .transport import control_transport


def _pack(ts):
    if ts is None or ts.shape is None:
        return None
    return (tuple(int(s) for s in ts.shape), torch_dtype_to_id(ts.dtype), bool(ts.requires_grad))


def _unpack(rec):
    ts = TensorStructure()
    if rec is not None:
        ts.shape = torch.Size(rec[0])
        ts.dtype = id_to_torch_dtype(rec[1])
        ts.requires_grad = rec[2]
    return ts


def broadcast_tensor_structure(input_tensor_structure, P_send, P_recv):
    """Structure of the tensor held by the root of each broadcast team, delivered
    to every member of that team.  A worker that only sends gets its own
    structure back."""
    ct = control_transport()
    out = input_tensor_structure
    teams = []
    if P_send.active:
        teams.append(("send", P_send))
    if P_recv.active and not (P_send.active and P_recv.ranks == P_send.ranks):
        teams.append(("recv", P_recv))
    # lowest root first on every worker: no cyclic wait
    teams.sort(key=lambda t: t[1].ranks[0])
    for kind, P in teams:
        payload = _pack(input_tensor_structure) if P.rank == 0 else None
        got = ct.broadcast_obj(payload, list(P.ranks), 0)
        if P.rank != 0:
            out = _unpack(got)
    return out


def _gather_shapes(local_tensor_structure, P_in, P_out=None):
    """{world rank: packed structure} for every member of P_in, known on P_in U P_out."""
    ct = control_transport()
    ranks = list(P_in.ranks)
    if P_out is not None:
        ranks += [r for r in P_out.ranks if r not in P_in.ranks]
    mine = _pack(local_tensor_structure) if P_in.active else None
    objs = ct.allgather_obj(mine, ranks)
    return {r: o for r, o in zip(ranks, objs) if r in P_in.ranks}


def assemble_global_tensor_structure(local_tensor_structure, P_in, P_out=None):
    """Structure of the global tensor whose pieces live on ``P_in`` (possibly
    unbalanced): along every dimension the local extents are summed over the
    workers of that grid line.  The result is also delivered to ``P_out``."""
    active_in = P_in.active
    active_out = P_out is not None and P_out.active
    ts = TensorStructure()
    if not (active_in or active_out):
        return ts
    recs = _gather_shapes(local_tensor_structure, P_in, P_out)
    shape = [int(s) for s in P_in.shape]
    first = recs[P_in.ranks[0]]
    ndim = len(first[0])
    if ndim != len(shape):
        raise ValueError("tensor rank and partition rank differ")
    table = np.zeros(shape + [ndim], dtype=int)
    for flat, idx in enumerate(range_index(shape)):
        table[idx] = recs[P_in.ranks[flat]][0]
    gshape = []
    for d in range(ndim):
        line = [0] * ndim
        total = 0
        for i in range(shape[d]):
            line[d] = i
            total += int(table[tuple(line)][d])
        gshape.append(total)
    ts.shape = torch.Size(gshape)
    ts.dtype = id_to_torch_dtype(first[1])
    ts.requires_grad = first[2]
    return ts


def assemble_global_tensor_structure_along_axis(local_tensor_structure, P_x, axis):
    """As above, but only ``axis`` is summed over the team ``P_x`` (the other
    extents are this worker's own)."""
    ts = TensorStructure()
    if not P_x.active:
        return ts
    recs = _gather_shapes(local_tensor_structure, P_x)
    gshape = [int(s) for s in local_tensor_structure.shape]
    gshape[axis] = sum(int(recs[r][0][axis]) for r in P_x.ranks)
    ts.shape = torch.Size(gshape)
    ts.dtype = local_tensor_structure.dtype
    ts.requires_grad = local_tensor_structure.requires_grad
    return ts
