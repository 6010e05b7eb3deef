"""Shared pieces of the primitive autograd Functions.

The seven data-movement primitives are written once, against the transport
interface of :mod:`distdl_b200.backends.common.transport`; a backend binds
them to its transport with :func:`bind_functional`.  (The reference writes
each primitive three times, once per backend:
``src/distdl/backends/{mpi_numpy,mpi_cupy,nccl_cupy}/functional``.)
"""
from __future__ import annotations

import types

from ....utilities.torch import zero_volume_tensor


class TransportBound:
    """Mixin: ``cls._transport`` is set by :func:`bind_functional`."""

    _transport = None

    @classmethod
    def transport(cls):
        if cls._transport is None:
            from .... import backends
            return backends.backend.transport()
        return cls._transport


def empty_output(reference, preserve_batch, device, dtype=None):
    """The zero-volume result of a worker that holds no output."""
    if preserve_batch and reference is not None and reference.dim() > 0:
        return zero_volume_tensor(reference.shape[0], dtype=dtype or reference.dtype, device=device)
    return zero_volume_tensor(dtype=dtype or (reference.dtype if reference is not None else None), device=device)


def scaled(grad, scale_backward):
    if scale_backward is None:
        return grad
    return grad / scale_backward


def bind_functional(transport, overrides=None):
    """Namespace with the Function classes of the seven primitives (and the accumulate form of the
    halo exchange) bound to ``transport``.
    ``overrides`` maps a class name to a replacement class (the native backend
    swaps in its fused-kernel versions)."""
    from . import all_gather, all_sum_reduce, broadcast, halo_exchange, reduce_scatter, repartition, sum_reduce
    ns = types.SimpleNamespace()
    for mod, name in ((broadcast, "BroadcastFunction"), (sum_reduce, "SumReduceFunction"),
                      (all_sum_reduce, "AllSumReduceFunction"), (all_gather, "AllGatherFunction"),
                      (reduce_scatter, "ReduceScatterFunction"), (repartition, "RepartitionFunction"),
                      (halo_exchange, "HaloExchangeFunction"), (halo_exchange, "HaloAccumulateFunction")):
        base = (overrides or {}).get(name) or getattr(mod, name)
        bound = type(name, (base,), {"_transport": transport})
        setattr(ns, name, bound)
    return ns
