"""Transport of the native backend.

CUDA tensors of a supported dtype move through this library's own kernels
(:mod:`distdl_b200.parallel.collectives`): one-shot / two-shot all-reduce,
all-gather, reduce-scatter and all-to-all that read and write the peers'
symmetric buffers directly over NVLink.  Anything else (CPU tensors, exotic
dtypes, teams that span more than one node) falls through to the NCCL
group transport.
"""
from __future__ import annotations

import torch

from ..common.transport import GroupTransport


class NativeTransport(GroupTransport):
    name = "native"
    recv_into = False      # its exchange kernel delivers into tensors of its own

    def __init__(self):
        super().__init__()
        self._coll = None

    def _collectives(self):
        if self._coll is None:
            from ...parallel import collectives
            self._coll = collectives
        return self._coll

    def prepare(self, ranks):
        import torch.distributed as dist
        if dist.is_initialized() and len(ranks) > 1 and torch.cuda.is_available():
            self._collectives().team(ranks)

    def _native_ok(self, t, ranks):
        return (t.is_cuda and len(ranks) > 1 and t.dtype in (torch.bfloat16, torch.float32, torch.float16)
                and self._collectives().available(ranks))

    def allreduce(self, tensor, ranks):
        if self._native_ok(tensor, ranks):
            return self._collectives().all_reduce(tensor, ranks)
        return super().allreduce(tensor, ranks)

    def allgather(self, tensor, ranks, shapes=None):
        if shapes is None and self._native_ok(tensor, ranks):
            return list(self._collectives().all_gather(tensor, ranks).unbind(0))
        return super().allgather(tensor, ranks, shapes)

    def reduce_scatter(self, chunks, ranks):
        if self._native_ok(chunks[0], ranks) and len({tuple(c.shape) for c in chunks}) == 1:
            return self._collectives().reduce_scatter(chunks, ranks)
        return super().reduce_scatter(chunks, ranks)

    def allgather_stacked(self, tensor, ranks):
        if self._native_ok(tensor, ranks):
            # parameter shards in the optimizer's peer-mapped buffer are read in place
            out = self._collectives().gather_in_place(tensor, ranks)
            if out is not None:
                return out
            return self._collectives().all_gather(tensor, ranks)
        return super().allgather_stacked(tensor, ranks)

    def reduce_scatter_stacked(self, stacked, ranks):
        if self._native_ok(stacked, ranks):
            return self._collectives().reduce_scatter(stacked, ranks)
        return super().reduce_scatter_stacked(stacked, ranks)

    def reduce_scatter_accumulate(self, stacked, acc, ranks, scale=1.0):
        """acc(fp32) += scale * reduce_scatter(stacked bf16); False when not applicable."""
        if not self._native_ok(stacked, ranks):
            return False
        return self._collectives().reduce_scatter_accumulate_(stacked, acc, ranks, scale)

    def box_plan(self, phases, team):
        """A :class:`distdl_b200.parallel.box_exchange.BoxPlan` for the strided boxes of a halo
        exchange or a repartition (packed, moved and unpacked by one kernel), or None when the
        team cannot use the peer-mapped memory (more than one node, no device)."""
        if not torch.cuda.is_available() or not 1 < len(team) <= 8 or not self._collectives().available(team):
            return None
        from ...parallel import box_exchange
        return box_exchange.BoxPlan(phases)

    def exchange(self, sends, recvs, team=None):
        """All messages of a team in one kernel.  Every member launches that kernel on every
        exchange, whatever its own messages are, because the kernel opens with a barrier over
        the team.  A message that does not fit a staging slot, or shares its ordered pair with
        another message, goes through the library's point-to-point path beside the kernel;
        that is decided per message from what both of its ends know
        (:func:`distdl_b200.parallel.collectives.exchange_split`)."""
        coll = self._collectives()
        if team is None or not torch.cuda.is_available() or not 1 < len(team) <= 8 or not coll.available(team):
            return super().exchange(sends, recvs, team)
        ok_s, ok_r = coll.exchange_split(len(team), coll.symm.heap().staging_bytes, sends, recvs)
        got = coll.exchange(team, [m for m, ok in zip(sends, ok_s) if ok], [m for m, ok in zip(recvs, ok_r) if ok])
        if all(ok_s) and all(ok_r):
            return got
        rest = super().exchange([m for m, ok in zip(sends, ok_s) if not ok],
                                [m for m, ok in zip(recvs, ok_r) if not ok], team)
        got, rest = iter(got), iter(rest)
        return [next(got) if ok else next(rest) for ok in ok_r]
