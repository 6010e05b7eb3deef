"""Partition algebra on six CPU ranks: factories, Cartesian grids, sub-teams, broadcast /
reduction team construction, equality, deactivation and the small collectives on Python data
(``src/distdl/backends/common/partition.py:19-1142`` in the reference)."""
import numpy as np
import pytest

from dist_harness import run_ranks


def body_factories(rank, world):
    import distdl_b200
    from distdl_b200.backends.common.world import PROC_NULL
    be = distdl_b200.backends.backend
    P_world = be.Partition()
    assert P_world.size == 6 and P_world.rank == rank and P_world.active and P_world.dim == 1
    assert list(P_world.shape) == [6] and int(P_world.index[0]) == rank
    # inclusive sub-team keeps the given ORDER; outsiders get an inactive partition
    P = P_world.create_partition_inclusive([4, 1, 2, 5])
    assert P.ranks == (4, 1, 2, 5) and P.size == 4
    if rank in (4, 1, 2, 5):
        assert P.active and P.rank == [4, 1, 2, 5].index(rank)
    else:
        assert not P.active and P.rank == PROC_NULL and P.index is None
    with pytest.raises(ValueError):
        P_world.create_partition_inclusive([1, 1])
    with pytest.raises(ValueError):
        P_world.create_partition_inclusive([0, 7])
    # Cartesian grid: row-major, must use all workers
    with pytest.raises(ValueError):
        P.create_cartesian_topology_partition([3, 2])
    C = P_world.create_partition_inclusive(range(6)).create_cartesian_topology_partition([2, 3])
    assert isinstance(C, be.CartesianPartition) and C.dim == 2 and list(C.shape) == [2, 3]
    assert list(C.index) == [rank // 3, rank % 3] and list(C.cartesian_index(4)) == [1, 1]
    assert C.cartesian_rank([1, 2]) == 5
    nb = C.neighbor_ranks(C.rank)
    i, j = rank // 3, rank % 3
    assert nb[0] == ((i - 1) * 3 + j if i > 0 else PROC_NULL, (i + 1) * 3 + j if i < 1 else PROC_NULL)
    assert nb[1] == (rank - 1 if j > 0 else PROC_NULL, rank + 1 if j < 2 else PROC_NULL)
    # sub-grids: keep a dimension, fix the others to my index
    row = C.create_cartesian_subtopology_partition([False, True])
    col = C.create_cartesian_subtopology_partition([True, False])
    assert row.ranks == tuple(range(i * 3, i * 3 + 3)) and list(row.shape) == [3]
    assert col.ranks == (j, j + 3) and list(col.shape) == [2]
    # all-reduction teams: vary only along the named axes, shape 1 elsewhere
    a0, a1 = C.create_allreduction_partition((0,)), C.create_allreduction_partition((1,))
    assert a0.ranks == (j, j + 3) and list(a0.shape) == [2, 1]
    assert a1.ranks == tuple(range(i * 3, i * 3 + 3)) and list(a1.shape) == [1, 3]
    assert C.create_allreduction_partition((0, 1)).ranks == tuple(range(6))
    with pytest.raises(ValueError):
        C.create_allreduction_partition((2,))
    # union: members of the first partition come first, duplicates once
    A, B = P_world.create_partition_inclusive([3, 4]), P_world.create_partition_inclusive([4, 0])
    U = A.create_partition_union(B)
    assert U.ranks == (3, 4, 0) and U.active == (rank in (3, 4, 0))
    # equality: same members, order, grid and activity
    assert C == P_world.create_partition_inclusive(range(6)).create_cartesian_topology_partition([2, 3])
    assert C != P_world.create_partition_inclusive(range(6)).create_cartesian_topology_partition([3, 2])
    assert A != B and A == P_world.create_partition_inclusive([3, 4])
    # deactivate: the worker drops out, the grid shape stays
    D = P_world.create_partition_inclusive(range(6)).create_cartesian_topology_partition([3, 2])
    D.deactivate()
    assert not D.active and D.rank == PROC_NULL and D.index is None and list(D.shape) == [3, 2]
    return True


def test_partition_factories_grids_and_subteams():
    run_ranks("test_partition", "body_factories", 6, timeout=180)


def body_send_recv_teams(rank, world):
    """create_broadcast_partition_to / create_reduction_partition_to: the source worker is rank 0 of
    the team it sends to; a worker is active in P_send only if it is such a root."""
    import distdl_b200
    be = distdl_b200.backends.backend
    P_world = be.Partition()
    P_src = P_world.create_partition_inclusive([4, 5]).create_cartesian_topology_partition([1, 2])
    P_dst = P_world.create_partition_inclusive([0, 1, 2, 3]).create_cartesian_topology_partition([2, 2])
    P_send, P_recv = P_src.create_broadcast_partition_to(P_dst)
    # source (0, j) -> destinations (0, j) and (1, j): ranks j and j + 2
    if rank in (4, 5):
        j = rank - 4
        assert P_send.active and P_send.rank == 0 and P_send.ranks == (rank, j, j + 2)
    else:
        assert not P_send.active
    if rank < 4:
        j = rank % 2
        assert P_recv.active and P_recv.ranks == (4 + j, j, j + 2) and P_recv.rank == 1 + rank // 2
    else:
        assert not P_recv.active
    # overlapping partitions: a root that is also a destination is in both teams
    P_src2 = P_world.create_partition_inclusive([0, 1]).create_cartesian_topology_partition([1, 2])
    S2, R2 = P_src2.create_broadcast_partition_to(P_dst)
    if rank in (0, 1):
        assert S2.active and S2.ranks[0] == rank and set(S2.ranks) == {rank, rank + 2}
    if rank < 4:
        assert R2.active and R2.ranks[0] == rank % 2
    # transposed source: [1, 2] read as [2, 1]
    S3, R3 = P_src2.create_broadcast_partition_to(P_dst, transpose_src=True)
    if rank < 4:
        assert R3.ranks[0] == rank // 2 and set(R3.ranks) == {rank // 2, 2 * (rank // 2), 2 * (rank // 2) + 1}
    # the reduction teams are the broadcast teams of the reverse direction
    P_a, P_b = P_dst.create_reduction_partition_to(P_src2)
    if rank < 4:
        assert P_a.active and P_a.ranks[0] == rank % 2
    # rule violations
    P_bad = P_world.create_partition_inclusive([0, 1, 2]).create_cartesian_topology_partition([3])
    with pytest.raises(Exception, match="No broadcast"):
        P_world.create_partition_inclusive([4, 5]).create_cartesian_topology_partition([2]) \
            .create_broadcast_partition_to(P_bad)
    with pytest.raises(Exception, match="No broadcast"):
        P_dst.create_broadcast_partition_to(P_src)                     # larger onto smaller
    return True


def test_broadcast_and_reduction_teams():
    run_ranks("test_partition", "body_send_recv_teams", 6, timeout=180)


def body_data_collectives(rank, world):
    import distdl_b200
    be = distdl_b200.backends.backend
    P_world = be.Partition()
    P = P_world.create_partition_inclusive([5, 3, 1])
    if not P.active:
        assert P.allgather_data(np.ones(2)) is None and P.allreduce_data(np.ones(2)) is None
        assert P.broadcast_data(np.ones(2)) is None
        return "outside"
    mine = np.array([P.rank + 1, 10 * (P.rank + 1)])
    got = P.allgather_data(mine)
    assert got.shape == (3, 2) and np.array_equal(got, np.array([[1, 10], [2, 20], [3, 30]]))
    assert np.array_equal(P.allreduce_data(mine), [6, 60])
    assert np.array_equal(P.allreduce_data(mine, op="prod"), [6, 6000])
    assert np.array_equal(P.allreduce_data(mine, op="max"), [3, 30])
    assert np.array_equal(P.allreduce_data(mine, op="min"), [1, 10])
    with pytest.raises(ValueError):
        P.allreduce_data(mine, op="xor")
    # broadcast from team rank 1 (world rank 3); arrays of any shape and dtype, and plain objects
    data = np.arange(6, dtype=np.float32).reshape(2, 3) * (rank + 1) if P.rank == 1 else None
    out = P.broadcast_data(data, root=1)
    assert out.dtype == np.float32 and np.array_equal(out, np.arange(6).reshape(2, 3) * 4)
    assert P.broadcast_data({"step": 7} if P.rank == 0 else None) == {"step": 7}
    # the source may be named through a sub-partition of the team
    P_sub = P_world.create_partition_inclusive([1])
    out = P.broadcast_data(np.array([42]) if rank == 1 else None, root=0, P_data=P_sub)
    assert int(out[0]) == 42
    with pytest.raises(ValueError):
        P.broadcast_data(None, root=0, P_data=P_world.create_partition_inclusive([0]))
    return "member"


def test_collectives_on_python_data():
    out = run_ranks("test_partition", "body_data_collectives", 6, timeout=180)
    assert out == ["outside", "member", "outside", "member", "outside", "member"]


def body_print_sequential(rank, world, path):
    """Rank-ordered output: every member appends its line when its turn comes."""
    import contextlib
    import io

    import distdl_b200
    P = distdl_b200.backends.backend.Partition()
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        P.print_sequential(f"hello from {rank}")
    with open(f"{path}/{rank}.txt", "w") as fh:
        fh.write(buf.getvalue())
    return buf.getvalue()


def test_print_sequential(tmp_path):
    out = run_ranks("test_partition", "body_print_sequential", 3, args=(str(tmp_path),), timeout=120)
    for r, text in enumerate(out):
        assert f"hello from {r}" in text and all(f"hello from {o}" not in text for o in range(3) if o != r)


def body_tensor_structures(rank, world):
    """Structure exchange: broadcast along send / receive teams, global shape of an UNBALANCED
    decomposition (also delivered to a second partition), the shape table, and the per-axis form."""
    import torch

    import distdl_b200
    from distdl_b200.utilities.torch import TensorStructure
    be = distdl_b200.backends.backend
    P_world = be.Partition()
    P = P_world.create_partition_inclusive([0, 1, 2, 3]).create_cartesian_topology_partition([2, 2])
    P_out = P_world.create_partition_inclusive([4, 5]).create_cartesian_topology_partition([1, 2])
    # unbalanced: row 0 has 3 rows, row 1 has 1; column 0 has 2 columns, column 1 has 5
    rows, cols = [3, 1], [2, 5]
    ts = TensorStructure()
    if P.active:
        t = torch.zeros(rows[int(P.index[0])], cols[int(P.index[1])], dtype=torch.float64, requires_grad=True)
        ts = TensorStructure(t)
    g = be.assemble_global_tensor_structure(ts, P, P_out)
    assert tuple(g.shape) == (4, 7) and g.dtype == torch.float64 and g.requires_grad
    table = be.tensor_decomposition.compute_subtensor_shapes_unbalanced(ts, P, P_out)
    assert table.shape == (2, 2, 2) and table[1, 0].tolist() == [1, 2] and table[0, 1].tolist() == [3, 5]
    if P.active:
        g1 = be.assemble_global_tensor_structure_along_axis(ts, P.create_allreduction_partition((1,)), 1)
        assert tuple(g1.shape) == (rows[int(P.index[0])], 7)
    # broadcast of the root's structure down its team
    P_src = P_world.create_partition_inclusive([4]).create_cartesian_topology_partition([1, 1])
    P_send, P_recv = P_src.create_broadcast_partition_to(P)
    mine = TensorStructure(torch.zeros(5, 2, dtype=torch.bfloat16)) if rank == 4 else TensorStructure()
    if P_send.active or P_recv.active:
        got = be.broadcast_tensor_structure(mine, P_send, P_recv)
        assert tuple(got.shape) == (5, 2) and got.dtype == torch.bfloat16 and not got.requires_grad
    return True


def test_tensor_structure_exchange():
    run_ranks("test_partition", "body_tensor_structures", 6, timeout=180)


def test_small_local_utilities():
    import torch

    from distdl_b200.utilities.index_tricks import cartesian_index_c, cartesian_index_f
    from distdl_b200.utilities.misc import Bunch, DummyContext, stream_barrier
    from distdl_b200.utilities.slicing import (assemble_index_filter, filtered_range_index, get_rearrange_ordering,
                                               range_index)
    from distdl_b200.utilities.torch import distdl_padding_to_torch_padding
    assert cartesian_index_c([2, 3], [1, 2]) == 5 and cartesian_index_f([2, 3], [1, 2]) == 5
    assert cartesian_index_c([2, 3], [1, 0]) == 3 and cartesian_index_f([2, 3], [1, 0]) == 1
    assert list(range_index([2, 2])) == [(0, 0), (0, 1), (1, 0), (1, 1)]
    # all indices of a 2 x 3 grid whose first entry is 1
    filt = assemble_index_filter((1, 0), [0])
    assert list(filtered_range_index([2, 3], filt)) == [(1, 0), (1, 1), (1, 2)]
    assert get_rearrange_ordering(3, 1) == ("p a b c", "a (p b) c")
    # per-dimension (left, right) pads -> torch.nn.functional.pad order (last dimension first)
    assert tuple(distdl_padding_to_torch_padding(np.array([[0, 0], [1, 2], [3, 4]]))) == (3, 4, 1, 2, 0, 0)
    b = Bunch(a=1)
    b.c = 2
    assert b.a == 1 and b["c"] == 2
    with pytest.raises(AttributeError):
        b.missing
    ctx = DummyContext()
    ctx.save_for_backward(torch.ones(1))
    assert len(ctx.saved_tensors) == 1
    stream_barrier(None)                                   # a no-op without a stream
