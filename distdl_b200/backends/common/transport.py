"""Data-plane transports: how a team of workers (an ordered tuple of world
ranks) moves tensors.  The seven primitives are written once against this
interface; a backend only chooses the transport.

``P2PTransport``
    Collectives composed from non-blocking point-to-point messages on one
    process group (gloo on CPU).  No sub-communicators are ever created, so
    there is no creation-order deadlock to guard against (the reference orders
    communicator creation by root rank for that reason,
    ``src/distdl/backends/common/partition.py:446-469``) and reductions add
    contributions in rank order, which makes CPU results reproducible.

``GroupTransport``
    Collectives of ``torch.distributed`` on cached sub-groups (NCCL on GPU):
    the baseline path and the fallback of the native backend.
"""
from __future__ import annotations

import pickle
import threading

import torch
import torch.distributed as dist

from . import world

# message tags (gloo matches on (source, tag); same-tag messages between one
# pair of ranks are delivered in order)
TAG_OBJ = 7001
TAG_BCAST = 7002
TAG_REDUCE = 7003
TAG_GATHER = 7004
TAG_SENDRECV = 7005


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(-1).view(torch.uint8)


def _recv_target(shape, dtype, into, device):
    """The tensor a message is received into: the caller's staging view if it fits, else a new one."""
    shape = tuple(int(v) for v in shape)
    if into and into[0] is not None:
        t = into[0]
        if tuple(t.shape) == shape and t.dtype == dtype and t.device.type == device.type and t.is_contiguous():
            return t
    return torch.empty(shape, dtype=dtype, device=device)


class P2PTransport:
    """Team collectives from isend/irecv on ``group`` (default: control-plane gloo group)."""

    recv_into = True       # exchange() accepts a target tensor as the fourth item of a receive
    name = "p2p"

    def __init__(self, group=None):
        self._group = group

    @property
    def group(self):
        return self._group if self._group is not None else world.control_group()

    # ---------------------------------------------------------------- low level
    def _isend(self, t, dst, tag):
        return dist.isend(_as_bytes(t), dst=dst, group=self.group, tag=tag)

    def _irecv_into(self, t, src, tag):
        return dist.irecv(t.view(-1).view(torch.uint8), src=src, group=self.group, tag=tag)

    def wire_tensor(self, t):
        """Tensor as this transport can carry it (CPU, contiguous)."""
        return t.detach().contiguous().cpu() if t.is_cuda else t.detach().contiguous()

    # ------------------------------------------------------------- collectives
    def broadcast(self, tensor, ranks, root_idx=0):
        """In place: ``tensor`` of ``ranks[root_idx]`` overwrites everyone's."""
        me = world.world_rank()
        if len(ranks) <= 1:
            return tensor
        buf = self.wire_tensor(tensor)
        root = ranks[root_idx]
        if me == root:
            reqs = [self._isend(buf, r, TAG_BCAST) for r in ranks if r != root]
            for q in reqs:
                q.wait()
        else:
            if not buf.is_contiguous() or buf is not tensor:
                buf = torch.empty(tensor.shape, dtype=tensor.dtype)
            self._irecv_into(buf, root, TAG_BCAST).wait()
            if buf is not tensor:
                tensor.copy_(buf)
        return tensor

    def reduce(self, tensor, ranks, root_idx=0):
        """Sum over the team, result on ``ranks[root_idx]`` only (returned there,
        ``None`` elsewhere).  Contributions are added in team-rank order."""
        me = world.world_rank()
        if len(ranks) <= 1:
            return tensor.clone()
        root = ranks[root_idx]
        buf = self.wire_tensor(tensor)
        if me != root:
            self._isend(buf, root, TAG_REDUCE).wait()
            return None
        parts = {}
        reqs = []
        for r in ranks:
            if r == root:
                continue
            parts[r] = torch.empty(buf.shape, dtype=buf.dtype)
            reqs.append(self._irecv_into(parts[r], r, TAG_REDUCE))
        for q in reqs:
            q.wait()
        acc_dtype = torch.float64 if buf.dtype == torch.float64 else (
            torch.float32 if buf.dtype.is_floating_point else buf.dtype)
        total = None
        for r in ranks:
            contrib = (buf if r == root else parts[r]).to(acc_dtype)
            total = contrib.clone() if total is None else total.add_(contrib)
        return total.to(buf.dtype).to(tensor.device)

    def allreduce(self, tensor, ranks):
        """Returns the team-wide sum (new tensor)."""
        if len(ranks) <= 1:
            return tensor.clone()
        out = self.reduce(tensor, ranks, 0)
        if out is None:
            out = torch.empty(tensor.shape, dtype=tensor.dtype)
        out = out.cpu() if out.is_cuda else out
        self.broadcast(out, ranks, 0)
        return out.to(tensor.device)

    def allgather(self, tensor, ranks, shapes=None):
        """List of every member's tensor in team-rank order.  ``shapes`` gives
        per-member shapes when they differ; default: all like mine."""
        me = world.world_rank()
        if len(ranks) <= 1:
            return [tensor.clone()]
        buf = self.wire_tensor(tensor)
        outs, reqs = [], []
        for i, r in enumerate(ranks):
            if r == me:
                outs.append(buf.clone())
            else:
                shp = buf.shape if shapes is None else tuple(shapes[i])
                outs.append(torch.empty(shp, dtype=buf.dtype))
                reqs.append(self._irecv_into(outs[-1], r, TAG_GATHER))
        reqs += [self._isend(buf, r, TAG_GATHER) for r in ranks if r != me]
        for q in reqs:
            q.wait()
        return [o.to(tensor.device) for o in outs]

    def reduce_scatter(self, chunks, ranks):
        """``chunks[i]`` is my contribution to member ``i``; returns the sum of
        everyone's contribution to me (added in team-rank order)."""
        me = world.world_rank()
        if len(ranks) <= 1:
            return chunks[0].clone()
        my_idx = ranks.index(me)
        device = chunks[my_idx].device
        bufs = [self.wire_tensor(c) for c in chunks]
        recv, reqs = {}, []
        for i, r in enumerate(ranks):
            if r == me:
                continue
            recv[i] = torch.empty(bufs[my_idx].shape, dtype=bufs[my_idx].dtype)
            reqs.append(self._irecv_into(recv[i], r, TAG_REDUCE))
        reqs += [self._isend(bufs[i], r, TAG_REDUCE) for i, r in enumerate(ranks) if r != me]
        for q in reqs:
            q.wait()
        dt = bufs[my_idx].dtype
        acc_dtype = torch.float64 if dt == torch.float64 else (torch.float32 if dt.is_floating_point else dt)
        total = None
        for i in range(len(ranks)):
            c = (bufs[my_idx] if i == my_idx else recv[i]).to(acc_dtype)
            total = c.clone() if total is None else total.add_(c)
        return total.to(dt).to(device)

    def allgather_stacked(self, tensor, ranks):
        """Equal shapes: ``[P, *shape]`` with every member's tensor."""
        return torch.stack(self.allgather(tensor, ranks))

    def reduce_scatter_stacked(self, stacked, ranks):
        """``stacked[i]`` is my contribution to member ``i`` (equal shapes)."""
        return self.reduce_scatter(list(stacked.unbind(0)), ranks)

    def exchange(self, sends, recvs, team=None):
        """Generic neighbour exchange (``team``: all workers that make this call together).
        ``sends`` = [(world_rank, tensor)], ``recvs`` = [(world_rank, shape, dtype)] or
        [(world_rank, shape, dtype, into)] -> list of received tensors (CPU or the transport's
        native device) in the order of ``recvs``; a message lands in ``into`` (a staging view of
        the caller's buffer manager) when that tensor has the message's shape, type and device."""
        outs, reqs = [], []
        for src, shape, dtype, *into in recvs:
            t = _recv_target(shape, dtype, into, torch.device("cpu"))
            outs.append(t)
            if t.numel():
                reqs.append(self._irecv_into(t, src, TAG_SENDRECV))
        keep = []
        for dst, t in sends:
            b = self.wire_tensor(t)
            keep.append(b)
            if b.numel():
                reqs.append(self._isend(b, dst, TAG_SENDRECV))
        for q in reqs:
            q.wait()
        return outs

    def barrier(self, ranks):
        if len(ranks) > 1:
            self.allreduce(torch.zeros(1), list(ranks))

    # --------------------------------------------------------- python objects
    def send_obj(self, obj, dst):
        payload = torch.frombuffer(bytearray(pickle.dumps(obj)), dtype=torch.uint8)
        n = torch.tensor([payload.numel()], dtype=torch.int64)
        dist.send(n, dst=dst, group=self.group, tag=TAG_OBJ)
        dist.send(payload, dst=dst, group=self.group, tag=TAG_OBJ)

    def recv_obj(self, src):
        n = torch.zeros(1, dtype=torch.int64)
        dist.recv(n, src=src, group=self.group, tag=TAG_OBJ)
        payload = torch.empty(int(n.item()), dtype=torch.uint8)
        dist.recv(payload, src=src, group=self.group, tag=TAG_OBJ)
        return pickle.loads(payload.numpy().tobytes())

    def allgather_obj(self, obj, ranks):
        me = world.world_rank()
        if len(ranks) <= 1:
            return [obj]
        root = ranks[0]
        if me == root:
            objs = [obj] + [self.recv_obj(r) for r in ranks[1:]]
            for r in ranks[1:]:
                self.send_obj(objs, r)
            return objs
        self.send_obj(obj, root)
        return self.recv_obj(root)

    def broadcast_obj(self, obj, ranks, root_idx=0):
        me = world.world_rank()
        if len(ranks) <= 1:
            return obj
        root = ranks[root_idx]
        if me == root:
            for r in ranks:
                if r != root:
                    self.send_obj(obj, r)
            return obj
        return self.recv_obj(root)


class GroupTransport(P2PTransport):
    """``torch.distributed`` collectives on cached sub-groups (NCCL for CUDA
    tensors).  Sub-groups are created by their members only and cached by rank
    tuple, as the reference caches NCCL communicators by the hash of the rank
    list (``src/distdl/backends/common/partition.py:128-146``)."""

    name = "group"
    _groups = {}
    _lock = threading.Lock()

    def __init__(self):
        super().__init__(None)

    def subgroup(self, ranks):
        key = tuple(sorted(int(r) for r in ranks))
        if len(key) == world.world_size():
            return dist.group.WORLD
        with self._lock:
            g = self._groups.get(key)
            if g is None:
                g = dist.new_group(list(key), use_local_synchronization=True)
                self._groups[key] = g
        return g

    @classmethod
    def clear_cache(cls):
        cls._groups.clear()

    def wire_tensor(self, t):
        return t.detach().contiguous()

    @staticmethod
    def _cuda(t):
        return t.is_cuda

    def broadcast(self, tensor, ranks, root_idx=0):
        if len(ranks) <= 1:
            return tensor
        if not tensor.is_cuda:
            return super().broadcast(tensor, ranks, root_idx)
        buf = tensor if tensor.is_contiguous() else tensor.contiguous()
        dist.broadcast(buf, src=ranks[root_idx], group=self.subgroup(ranks))
        if buf is not tensor:
            tensor.copy_(buf)
        return tensor

    def reduce(self, tensor, ranks, root_idx=0):
        if len(ranks) <= 1:
            return tensor.clone()
        if not tensor.is_cuda:
            return super().reduce(tensor, ranks, root_idx)
        out = tensor.detach().clone().contiguous()
        dist.reduce(out, dst=ranks[root_idx], group=self.subgroup(ranks))
        return out if world.world_rank() == ranks[root_idx] else None

    def allreduce(self, tensor, ranks):
        if len(ranks) <= 1:
            return tensor.clone()
        if not tensor.is_cuda:
            return super().allreduce(tensor, ranks)
        out = tensor.detach().clone().contiguous()
        dist.all_reduce(out, group=self.subgroup(ranks))
        return out

    def allgather(self, tensor, ranks, shapes=None):
        if len(ranks) <= 1:
            return [tensor.clone()]
        if not tensor.is_cuda or shapes is not None or list(ranks) != sorted(ranks):
            if tensor.is_cuda:
                return self._allgather_p2p_cuda(tensor, ranks, shapes)
            return super().allgather(tensor, ranks, shapes)
        buf = tensor.detach().contiguous()
        out = torch.empty((len(ranks),) + tuple(buf.shape), dtype=buf.dtype, device=buf.device)
        dist.all_gather_into_tensor(out, buf, group=self.subgroup(ranks))
        return list(out.unbind(0))

    def _allgather_p2p_cuda(self, tensor, ranks, shapes):
        me = world.world_rank()
        buf = tensor.detach().contiguous()
        outs, ops = [], []
        for i, r in enumerate(ranks):
            if r == me:
                outs.append(buf.clone())
            else:
                shp = buf.shape if shapes is None else tuple(shapes[i])
                outs.append(torch.empty(shp, dtype=buf.dtype, device=buf.device))
                if outs[-1].numel():
                    ops.append(dist.P2POp(dist.irecv, outs[-1], r))
                if buf.numel():
                    ops.append(dist.P2POp(dist.isend, buf, r))
        if ops:
            for q in dist.batch_isend_irecv(ops):
                q.wait()
        return outs

    def reduce_scatter(self, chunks, ranks):
        if len(ranks) <= 1:
            return chunks[0].clone()
        if not chunks[0].is_cuda or list(ranks) != sorted(ranks):
            if chunks[0].is_cuda:
                me = world.world_rank()
                stacked = torch.stack([c.contiguous() for c in chunks])
                dist.all_reduce(stacked, group=self.subgroup(ranks))
                return stacked[list(ranks).index(me)].clone()
            return super().reduce_scatter(chunks, ranks)
        inp = torch.stack([c.contiguous() for c in chunks])
        out = torch.empty_like(inp[0])
        dist.reduce_scatter_tensor(out, inp, group=self.subgroup(ranks))
        return out

    def exchange(self, sends, recvs, team=None):
        cuda = any(t.is_cuda for _, t in sends) or (torch.cuda.is_available() and dist.get_backend() == "nccl")
        if not cuda:
            return super().exchange(sends, recvs, team)
        dev = torch.device("cuda", torch.cuda.current_device())
        outs, ops, keep = [], [], []
        for src, shape, dtype, *into in recvs:
            t = _recv_target(shape, dtype, into, dev)
            outs.append(t)
            if t.numel():
                ops.append(dist.P2POp(dist.irecv, t, src))
        for dst, t in sends:
            b = t.detach().contiguous()
            keep.append(b)
            if b.numel():
                ops.append(dist.P2POp(dist.isend, b, dst))
        if ops:
            for q in dist.batch_isend_irecv(ops):
                q.wait()
        return outs

    def barrier(self, ranks):
        if len(ranks) > 1:
            if torch.cuda.is_available() and dist.get_backend() == "nccl":
                dist.barrier(group=self.subgroup(ranks))
            else:
                super().barrier(ranks)


_control = None


def control_transport() -> P2PTransport:
    """Transport of the control plane (metadata): p2p over the gloo group."""
    global _control
    if _control is None:
        _control = P2PTransport()
    return _control
