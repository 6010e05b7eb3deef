"""Partitions: teams of workers, optionally arranged on a Cartesian grid.

"The form of parallelism is induced by the partitioning of the tensors": every
layer of the framework is parameterised by partitions.  The reference builds
them from MPI communicators and groups
(``src/distdl/backends/common/partition.py:19`` ``MPIPartition``, ``:976``
``MPICartesianPartition``).  Here a partition is a plain value object -- an
ordered tuple of world ranks plus a grid shape -- and every factory below is
*local arithmetic on rank lists*: no communicator is created, no collective is
run, and nothing can deadlock while partitions are being derived.  Process
groups (NCCL) or symmetric-memory teams (native backend) are attached lazily by
the transports when data actually moves.

Differences from the reference that follow from this design:

* an inactive worker (one that is not a member) still knows the member list
  and the grid shape, so ``size``/``shape`` stay meaningful on it; ``rank`` is
  ``PROC_NULL`` and ``index`` is ``None`` there;
* ``create_*`` methods are not collective; calling them on a subset of the
  workers is harmless.
"""
from __future__ import annotations

import numpy as np
import torch

from ...utilities.index_tricks import cartesian_index_c, cartesian_index_f
from ...utilities.slicing import assemble_index_filter, filtered_range_index, range_index
from . import world
from .transport import control_transport

PROC_NULL = world.PROC_NULL


def _default_device():
    if torch.cuda.is_available():
        from ... import config
        if config.array_is_device():
            return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def _global_setup():
    if world.world_size() <= 1:
        return
    world.control_group()
    from ... import backends
    be = backends.backend
    if be is not None and getattr(be, "name", "") == "native_cupy" and torch.cuda.is_available():
        from ...parallel import symm
        symm.heap()


class Partition:
    """An ordered team of workers.

    Parameters
    ----------
    ranks : iterable of int, optional
        World ranks of the members in team order.  ``None`` means every process
        of the job (the world partition).  An empty list gives a null partition.
    root : tuple, optional
        Identity of the ancestor partition (its rank tuple); unions are only
        allowed between partitions with the same root.
    device : torch.device, optional
        Where this worker's tensors live.
    """

    def __init__(self, ranks=None, root=None, device=None, requested_device=None, initialize_backend_comm=False):
        if ranks is None:
            ranks = range(world.world_size())
            # Building the world partition is the one point every process is
            # known to reach: set up what needs all of them (the control-plane
            # group; the symmetric heap of the native backend).
            _global_setup()
        self.ranks = tuple(int(r) for r in ranks)
        if len(set(self.ranks)) != len(self.ranks):
            raise ValueError("duplicate ranks in partition")
        me = world.world_rank()
        self.active = me in self.ranks
        self.rank = self.ranks.index(me) if self.active else PROC_NULL
        self.size = len(self.ranks)
        self._root = tuple(root) if root is not None else self.ranks
        self.shape = np.array([self.size], dtype=int)
        self.dim = 1
        self.index = np.array([self.rank], dtype=int) if self.active else None
        if requested_device is not None and device is None:
            device = torch.device(requested_device) if not isinstance(requested_device, torch.device) \
                else requested_device
        self.device = device if device is not None else _default_device()
        self._backend_ready = False
        if initialize_backend_comm:
            self.initialize_backend_comm()

    # ------------------------------------------------------------------ basics
    def __repr__(self):
        return (f"{type(self).__name__}(ranks={self.ranks}, shape={self.shape.tolist()}, "
                f"rank={self.rank}, active={self.active})")

    def __eq__(self, other):
        if not isinstance(other, Partition):
            return NotImplemented
        return (self.ranks == other.ranks and self.dim == other.dim
                and np.array_equal(self.shape, other.shape) and self.active == other.active
                and str(self.device) == str(other.device))

    __hash__ = None

    def initialize_backend_comm(self):
        """Attaches whatever the active backend needs to move data inside this
        team (an NCCL sub-group, or nothing for the p2p / symmetric-memory
        transports).  Only members take part."""
        if self.active and not self._backend_ready and self.size > 1:
            from ... import backends
            be = backends.backend
            if be is not None and hasattr(be, "prepare_team"):
                be.prepare_team(self.ranks)
        self._backend_ready = True

    def deactivate(self):
        """Marks the partition unusable for this worker (frees nothing: there
        are no communicator handles to free)."""
        self.active = False
        self.rank = PROC_NULL
        self.index = None

    def barrier(self):
        if self.active:
            control_transport().barrier(list(self.ranks))

    def print_sequential(self, val):
        from ...utilities.debug import print_sequential
        print_sequential(self, val)

    def set_device(self):
        from ... import backends
        return backends.backend.set_device(rank=world.world_rank())

    # --------------------------------------------------------------- factories
    def _make(self, ranks, shape=None):
        if shape is None:
            return Partition(ranks, root=self._root, device=self.device)
        return CartesianPartition(ranks, shape, root=self._root, device=self.device)

    def create_partition_inclusive(self, ranks):
        """Team made of the members with the given *team* ranks, in that order."""
        ranks = [int(r) for r in np.asarray(ranks).reshape(-1)]
        for r in ranks:
            if r < 0 or r >= self.size:
                raise ValueError(f"rank {r} outside partition of size {self.size}")
        return self._make([self.ranks[r] for r in ranks])

    def create_partition_union(self, other, initialize_backend_comm=False):
        """Members of ``self`` first, then those of ``other`` not already present."""
        if self._root != other._root:
            raise Exception("Cannot create union: partitions do not share a root.")
        seen = set(self.ranks)
        merged = list(self.ranks) + [r for r in other.ranks if r not in seen]
        P = self._make(merged)
        if initialize_backend_comm:
            P.initialize_backend_comm()
        return P

    def create_cartesian_topology_partition(self, shape, **options):
        """Same team, arranged row-major on a grid of the given shape."""
        shape = [int(s) for s in np.asarray(shape).reshape(-1)]
        if int(np.prod(shape)) != self.size:
            raise ValueError(f"Cartesian shape {shape} does not use all {self.size} workers")
        return self._make(self.ranks, shape)

    # -------------------------------------------------- broadcast / reduction
    @staticmethod
    def _grid(P):
        """(shape, {world rank: index}) of a partition; unstructured ones are 1-D."""
        shape = [int(s) for s in P.shape]
        table = {}
        for flat, idx in enumerate(range_index(shape)):
            table[P.ranks[flat]] = idx
        return shape, table

    def _broadcast_groups(self, P_dest, transpose_src, transpose_dest):
        """For the broadcast rules: {colour: (root world rank, [dest world ranks])}."""
        P_src = self
        src_shape, src_tab = self._grid(P_src)
        dest_shape, dest_tab = self._grid(P_dest)
        src_dim, dest_dim = len(src_shape), len(dest_shape)
        if src_dim > dest_dim:
            raise Exception("No broadcast: Source partition larger than destination partition.")
        s = [1] * dest_dim
        s[dest_dim - src_dim:] = src_shape[::-1] if transpose_src else src_shape
        d = dest_shape[::-1] if transpose_dest else dest_shape
        for a, b in zip(s, d):
            if a != b and a != 1:
                raise Exception("No broadcast: Dimensions don't match or source is not 1 where there is a mismatch.")
        match = [k for k in range(dest_dim) if s[k] == d[k]]
        src_colour = {}
        for r, idx in src_tab.items():
            full = [0] * dest_dim
            full[dest_dim - src_dim:] = list(idx)[::-1] if transpose_src else list(idx)
            fn = cartesian_index_f if transpose_src else cartesian_index_c
            src_colour[r] = fn([s[k] for k in match], [full[k] for k in match])
        dest_colour = {}
        for r, idx in dest_tab.items():
            full = list(idx)[::-1] if transpose_dest else list(idx)
            fn = cartesian_index_f if transpose_dest else cartesian_index_c
            dest_colour[r] = fn([d[k] for k in match], [full[k] for k in match])
        groups = {}
        for r in P_src.ranks:
            c = src_colour[r]
            if c in groups:
                raise Exception("No broadcast: two source workers map to the same destination set.")
            groups[c] = (r, [q for q in P_dest.ranks if dest_colour[q] == c])
        return groups, src_colour, dest_colour

    def create_broadcast_partition_to(self, P_dest, transpose_src=False, transpose_dest=False,
                                      initialize_backend_comm=False):
        """Teams for broadcasting from ``self`` to ``P_dest`` under the broadcast
        rules (source dims, left-padded with ones, must equal the destination's
        or be 1).  Returns ``(P_send, P_recv)``: the team this worker is the
        root of (if it is a source) and the team it receives in (if it is a
        destination); either may be inactive, and they may be the same team.
        The root is always team rank 0."""
        null = Partition([], root=self._root, device=self.device)
        if self._root != P_dest._root:
            raise Exception("Cannot create union: partitions do not share a root.")
        me = world.world_rank()
        in_src, in_dest = me in self.ranks, me in P_dest.ranks
        # pure arithmetic on rank lists: workers outside both partitions check the rules as well, so
        # that a violation raises on every worker and not only on the members
        groups, src_colour, dest_colour = self._broadcast_groups(P_dest, transpose_src, transpose_dest)
        if not (in_src or in_dest):
            return null, null
        P_send, P_recv = null, null
        if in_src:
            root, dests = groups[src_colour[me]]
            P_send = self._make([root] + [q for q in dests if q != root])
        if in_dest:
            root, dests = groups[dest_colour[me]]
            team = [root] + [q for q in dests if q != root]
            P_recv = P_send if (in_src and tuple(team) == P_send.ranks) else self._make(team)
        if initialize_backend_comm:
            # lowest root first, so that two workers never wait on each other's
            # team while holding their own
            for P in sorted([P_send, P_recv], key=lambda p: p.ranks[0] if p.ranks else -1):
                P.initialize_backend_comm()
        return P_send, P_recv

    def create_reduction_partition_to(self, P_dest, transpose_src=False, transpose_dest=False,
                                      initialize_backend_comm=False):
        """Mirror of :meth:`create_broadcast_partition_to`: ``self`` is the large
        partition being reduced onto ``P_dest``.  Returns ``(P_send, P_recv)``:
        the team this worker contributes in, and the team it is the root
        (receiver) of.  The root is team rank 0."""
        root_team, member_team = P_dest.create_broadcast_partition_to(
            self, transpose_src=transpose_dest, transpose_dest=transpose_src,
            initialize_backend_comm=initialize_backend_comm)
        # In the broadcast picture P_dest's workers are the roots of their teams;
        # for a reduction the root receives and the members send.
        return member_team, root_team

    def create_allreduction_partition(self, axes_reduce, initialize_backend_comm=False):
        """Sub-team of the workers whose index differs from mine only along
        ``axes_reduce``; shape is the partition's shape along those axes and 1 elsewhere."""
        if not self.active:
            return Partition([], root=self._root, device=self.device)
        axes = [int(a) for a in axes_reduce]
        for a in axes:
            if a >= self.dim:
                raise ValueError(f"Dimension {a} in axes_reduce exceeds partition dimesion.")
        shape = [int(self.shape[k]) if k in axes else 1 for k in range(self.dim)]
        filt = assemble_index_filter(tuple(int(i) for i in self.index), axes, invert=True)
        full_shape = [int(s) for s in self.shape]
        members = [self.ranks[cartesian_index_c(full_shape, idx)] for idx in filtered_range_index(full_shape, filt)]
        P = self._make(members, shape)
        if initialize_backend_comm:
            P.initialize_backend_comm()
        return P

    # -------------------------------------------------- python-data collectives
    def broadcast_data(self, data, root=0, P_data=None):
        """Ships a small array (or any picklable object) from one member to all.

        With ``P_data`` the source is rank ``root`` of that sub-partition (whose
        members must all be members of ``self``).  Returns the data on every member."""
        if not self.active:
            return None
        if P_data is not None:
            if len(P_data.ranks) == 0:
                raise ValueError("P_data has no members")
            src_world = P_data.ranks[root]
        else:
            src_world = self.ranks[root]
        if src_world not in self.ranks:
            raise ValueError("broadcast source is not a member of the partition")
        out = control_transport().broadcast_obj(data, list(self.ranks), self.ranks.index(src_world))
        return out

    def allgather_data(self, data):
        """Stacks one equally-shaped array per member along a new leading axis."""
        if not self.active:
            return None
        objs = control_transport().allgather_obj(np.asarray(data), list(self.ranks))
        return np.stack([np.asarray(o) for o in objs])

    def allreduce_data(self, data, op="sum"):
        """Element-wise reduction of one array per member; ``op`` in sum/prod/max/min."""
        if not self.active:
            return None
        fn = {"sum": np.sum, "prod": np.prod, "max": np.max, "min": np.min}.get(op)
        if fn is None:
            raise ValueError(f"unsupported reduction {op!r}")
        objs = control_transport().allgather_obj(np.asarray(data), list(self.ranks))
        return fn(np.stack([np.asarray(o) for o in objs]), axis=0)

    # neighbours of an unstructured team: none
    def cartesian_index(self, rank):
        return np.array([int(rank)], dtype=int)


class CartesianPartition(Partition):
    """A team arranged row-major on a grid (last grid index varies fastest)."""

    def __init__(self, ranks, shape, root=None, device=None, requested_device=None):
        super().__init__(ranks, root=root, device=device, requested_device=requested_device)
        self.shape = np.asarray([int(s) for s in shape], dtype=int)
        self.dim = len(self.shape)
        if self.size and int(np.prod(self.shape)) != self.size:
            raise ValueError("grid shape does not match the number of workers")
        self.index = self.cartesian_index(self.rank) if self.active else None

    def deactivate(self):
        super().deactivate()  # the grid shape is kept

    def cartesian_index(self, rank):
        """Grid index of a team rank."""
        if rank is None or rank < 0:
            return None
        return np.asarray(np.unravel_index(int(rank), tuple(int(s) for s in self.shape)), dtype=int)

    def cartesian_rank(self, index):
        return cartesian_index_c([int(s) for s in self.shape], [int(i) for i in index])

    def create_cartesian_subtopology_partition(self, remain_shape):
        """Keeps the grid dimensions flagged in ``remain_shape``; the others are
        fixed to this worker's index (one sub-grid per combination)."""
        if not self.active:
            return Partition([], root=self._root, device=self.device)
        keep = [bool(k) for k in remain_shape]
        if len(keep) != self.dim:
            raise ValueError("remain_shape must have one flag per grid dimension")
        dims = [k for k in range(self.dim) if keep[k]]
        filt = assemble_index_filter(tuple(int(i) for i in self.index), dims, invert=True)
        full = [int(s) for s in self.shape]
        members = [self.ranks[cartesian_index_c(full, idx)] for idx in filtered_range_index(full, filt)]
        return self._make(members, [full[k] for k in dims] or [1])

    def neighbor_ranks(self, rank):
        """Per grid dimension, the team ranks of the (left, right) neighbours of
        ``rank``; ``PROC_NULL`` beyond the edges."""
        idx = [int(i) for i in self.cartesian_index(rank)]
        out = []
        for d in range(self.dim):
            pair = []
            for step in (-1, 1):
                j = list(idx)
                j[d] += step
                pair.append(self.cartesian_rank(j) if 0 <= j[d] < int(self.shape[d]) else PROC_NULL)
            out.append(tuple(pair))
        return out


# Names used by the reference's backends
MPIPartition = Partition
MPICartesianPartition = CartesianPartition
