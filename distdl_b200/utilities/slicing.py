"""Index arithmetic for tensors split over Cartesian partitions.

The decomposition rule is the *balanced* one of the reference
(``src/distdl/utilities/slicing.py:8-51``): an extent ``n`` split over ``P``
workers gives every worker ``n // P`` entries and the first ``n % P`` workers one
more.  All functions accept scalars, sequences or arrays and return NumPy
``int64`` arrays (or tuples of ``slice``), so they compose with partition
shapes and indices directly.
"""
from __future__ import annotations

import itertools

import numpy as np

INDEX_DTYPE = np.int64
MAX_INT = np.iinfo(INDEX_DTYPE).max
MIN_INT = np.iinfo(INDEX_DTYPE).min


def _arr(v):
    return np.atleast_1d(np.asarray(v, dtype=INDEX_DTYPE))


def compute_subshape(P_shape, index, shape):
    """Local shape of the sub-tensor owned by the worker at ``index``."""
    P, i, n = _arr(P_shape), _arr(index), _arr(shape)
    base, extra = np.divmod(n, P)
    return base + (i < extra).astype(INDEX_DTYPE)


def compute_subshape_along_axis(P_shape, index, shape, axis):
    """As :func:`compute_subshape`, but only ``axis`` is split; other extents are kept."""
    P, i, n = _arr(P_shape), _arr(index), _arr(shape)
    out = n.copy()
    for ax in np.atleast_1d(axis):
        base, extra = divmod(int(n[ax]), int(P[ax]))
        out[ax] = base + (1 if int(i[ax]) < extra else 0)
    return out


def compute_start_index(P_shape, index, shape):
    """Global index of the first entry owned by the worker at ``index``."""
    P, i, n = _arr(P_shape), _arr(index), _arr(shape)
    base, extra = np.divmod(n, P)
    return base * i + np.minimum(i, extra)


def compute_stop_index(P_shape, index, shape):
    """One past the last global index owned by the worker at ``index``."""
    return compute_start_index(P_shape, index, shape) + compute_subshape(P_shape, index, shape)


def compute_intersection(r0_start_index, r0_stop_index, r1_start_index, r1_stop_index):
    """Overlap of two index boxes: (start, stop, shape); empty dims have extent 0."""
    lo = np.maximum(_arr(r0_start_index), _arr(r1_start_index))
    hi = np.minimum(_arr(r0_stop_index), _arr(r1_stop_index))
    return lo, hi, np.maximum(hi - lo, 0)


def assemble_slices(start_index, stop_index):
    """Tuple of ``slice(start, stop)`` per dimension."""
    return tuple(slice(int(a), int(b), None) for a, b in zip(_arr(start_index), _arr(stop_index)))


def compute_partition_intersection(P_x_r_shape, P_x_r_index, P_x_s_shape, P_x_s_index, x_shape):
    """Slices, relative to worker *r*'s sub-tensor, of the region it shares with
    worker *s* when the same global tensor is split by two partitions; ``None``
    when they share nothing."""
    r_lo = compute_start_index(P_x_r_shape, P_x_r_index, x_shape)
    r_hi = compute_stop_index(P_x_r_shape, P_x_r_index, x_shape)
    s_lo = compute_start_index(P_x_s_shape, P_x_s_index, x_shape)
    s_hi = compute_stop_index(P_x_s_shape, P_x_s_index, x_shape)
    lo, _, extent = compute_intersection(r_lo, r_hi, s_lo, s_hi)
    if int(np.prod(extent)) == 0:
        return None
    rel = lo - r_lo
    return assemble_slices(rel, rel + extent)


def compute_nd_slice_volume(slices):
    return int(np.prod([s.stop - s.start for s in slices]))


def compute_nd_slice_shape(slices):
    """Shape of the box described by a tuple of slices."""
    return tuple(int(s.stop - s.start) for s in slices)


def range_index(shape):
    """Row-major iterator over all Cartesian indices of ``shape``."""
    yield from itertools.product(*(range(int(n)) for n in shape))


def worker_layout(shape):
    """Array of ``shape`` whose entries are the row-major worker ranks."""
    dims = [int(n) for n in np.atleast_1d(shape)]
    return np.arange(int(np.prod(dims)), dtype=int).reshape(dims)


def filtered_range_index(shape, filter):
    """Row-major iterator over the indices of ``shape`` that match ``filter``
    (an index with ``None`` for "any")."""
    ranges = [range(int(n)) if f is None else ([int(f)] if 0 <= int(f) < int(n) else [])
              for n, f in zip(shape, filter)]
    yield from itertools.product(*ranges)


def assemble_index_filter(index, dims, invert=False):
    """Filter for :func:`filtered_range_index`: keeps ``index[k]`` for ``k`` in
    ``dims`` (or for ``k`` not in ``dims`` when ``invert``), ``None`` elsewhere."""
    dims = set(int(d) for d in dims)
    return tuple(index[k] if ((k in dims) != bool(invert)) else None for k in range(len(index)))


def get_rearrange_ordering(num_dims, axis):
    """einops patterns moving a leading worker dimension ``p`` into ``axis``:
    ``('p a b c', 'a (p b) c')`` for ``num_dims=3, axis=1``."""
    names = [chr(ord("a") + k) for k in range(num_dims)]
    merged = list(names)
    merged[axis] = f"(p {names[axis]})"
    return "p " + " ".join(names), " ".join(merged)
