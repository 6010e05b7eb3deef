"""Adjoint and value tests of the seven primitives on CPU ranks (gloo)."""
import numpy as np
import pytest
import torch

from dist_harness import run_ranks


def _P(world_ranks, shape):
    import distdl_b200 as d
    P_world = d.backends.backend.Partition()
    P_base = P_world.create_partition_inclusive(world_ranks)
    return P_base.create_cartesian_topology_partition(shape)


# ------------------------------------------------------------------ broadcast
def body_broadcast(rank, world, P_x_ranks, P_x_shape, P_y_ranks, P_y_shape, tsrc, tdst, x_shape):
    from adjoint_test import check_adjoint_test_tight
    from distdl_b200.nn import Broadcast
    from distdl_b200.utilities.torch import zero_volume_tensor
    torch.manual_seed(rank)
    P_x, P_y = _P(P_x_ranks, P_x_shape), _P(P_y_ranks, P_y_shape)
    layer = Broadcast(P_x, P_y, transpose_src=tsrc, transpose_dest=tdst, preserve_batch=False)
    x = zero_volume_tensor()
    if P_x.active:
        x = torch.randn(*x_shape, dtype=torch.float64)
    x.requires_grad = True
    y = layer(x)
    dy = zero_volume_tensor()
    if P_y.active:
        assert tuple(y.shape) == tuple(x_shape)
        dy = torch.randn(*x_shape, dtype=torch.float64)
    y.backward(dy)
    dx = x.grad
    check_adjoint_test_tight(x.detach(), dx, y.detach(), dy)
    return True


BCAST_CASES = [
    # P_x ranks, shape, P_y ranks, shape, transpose_src, transpose_dest, x shape
    ([0], [1], [0, 1, 2, 3], [2, 2], False, False, [3, 5]),
    ([0, 1], [1, 2], [0, 1, 2, 3], [2, 2], False, False, [3, 5]),
    ([0, 1], [2, 1], [0, 1, 2, 3], [2, 2], False, False, [4, 2]),
    ([0, 1], [2], [2, 3, 0, 1], [2, 2], False, False, [4]),      # disjoint-ish ordering
    ([2, 3], [2], [0, 1, 2, 3], [2, 2], False, False, [4]),      # overlapping, roots not first
    ([0, 1], [1, 2], [0, 1, 2, 3], [2, 2], True, False, [3]),    # transposed source
    ([0, 1, 2, 3], [2, 2], [0, 1, 2, 3], [2, 2], False, False, [3]),  # identity
    ([0], [1], [1, 2], [2], False, False, [6]),                  # disjoint
]


@pytest.mark.parametrize("case", BCAST_CASES)
def test_broadcast_adjoint(case):
    run_ranks("test_primitives", "body_broadcast", 4, case)


def body_sum_reduce(rank, world, P_x_ranks, P_x_shape, P_y_ranks, P_y_shape, tsrc, tdst, x_shape):
    from adjoint_test import check_adjoint_test_tight
    from distdl_b200.nn import SumReduce
    from distdl_b200.utilities.torch import zero_volume_tensor
    torch.manual_seed(rank)
    P_x, P_y = _P(P_x_ranks, P_x_shape), _P(P_y_ranks, P_y_shape)
    layer = SumReduce(P_x, P_y, transpose_src=tsrc, transpose_dest=tdst, preserve_batch=False)
    x = zero_volume_tensor()
    if P_x.active:
        x = torch.randn(*x_shape, dtype=torch.float64)
    x.requires_grad = True
    y = layer(x)
    dy = zero_volume_tensor()
    if P_y.active:
        assert tuple(y.shape) == tuple(x_shape)
        dy = torch.randn(*x_shape, dtype=torch.float64)
    y.backward(dy)
    check_adjoint_test_tight(x.detach(), x.grad, y.detach(), dy)
    return True


@pytest.mark.parametrize("case", [
    ([0, 1, 2, 3], [2, 2], [0], [1], False, False, [3, 5]),
    ([0, 1, 2, 3], [2, 2], [0, 1], [1, 2], False, False, [3, 5]),
    ([0, 1, 2, 3], [2, 2], [2, 3], [2, 1], False, False, [3]),
    ([0, 1, 2, 3], [2, 2], [0, 1], [1, 2], False, True, [3]),
    ([1, 2], [2], [0], [1], False, False, [6]),
])
def test_sum_reduce_adjoint(case):
    run_ranks("test_primitives", "body_sum_reduce", 4, case)


# ------------------------------------------------- all-reduce / gather / scatter
def body_team_collectives(rank, world):
    from adjoint_test import check_adjoint_test_tight
    from distdl_b200.nn import AllGather, AllSumReduce, ReduceScatter
    torch.manual_seed(100 + rank)
    P = _P([0, 1, 2, 3], [2, 2])
    # AllSumReduce over axis 1: rows {0,1} and {2,3}
    layer = AllSumReduce(P, axes_reduce=(1,))
    x = torch.randn(3, 4, dtype=torch.float64, requires_grad=True)
    y = layer(x)
    dy = torch.randn(3, 4, dtype=torch.float64)
    y.backward(dy)
    check_adjoint_test_tight(x.detach(), x.grad, y.detach(), dy)
    # value check: ranks in one row agree
    import torch.distributed as dist
    rows = [torch.zeros(3, 4, dtype=torch.float64) for _ in range(4)]
    dist.all_gather(rows, y.detach())
    assert torch.allclose(rows[0], rows[1]) and torch.allclose(rows[2], rows[3])
    assert not torch.allclose(rows[0], rows[2])

    # AllGather along tensor axis 1 with an uneven global extent (7 over 2 workers)
    ext = 4 if P.index[1] == 0 else 3
    ag = AllGather(P, axes_all_gather=(1,))
    x = torch.randn(5, ext, dtype=torch.float64, requires_grad=True)
    y = ag(x)
    assert tuple(y.shape) == (5, 7)
    dy = torch.randn(5, 7, dtype=torch.float64)
    y.backward(dy)
    check_adjoint_test_tight(x.detach(), x.grad, y.detach(), dy)
    assert torch.equal(y.detach()[:, :4] if P.index[1] == 0 else y.detach()[:, 4:], x.detach())

    # ReduceScatter along axis 0 (9 rows over 2 workers -> 5 / 4)
    rs = ReduceScatter(P, axes_reduce_scatter=(0,))
    x = torch.randn(9, 3, dtype=torch.float64, requires_grad=True)
    y = rs(x)
    assert tuple(y.shape) == ((5, 3) if P.index[0] == 0 else (4, 3))
    dy = torch.randn(*y.shape, dtype=torch.float64)
    y.backward(dy)
    check_adjoint_test_tight(x.detach(), x.grad, y.detach(), dy)
    # scale_backward divides the gradient
    layer = AllSumReduce(P, axes_reduce=(0, 1), scale_backward=4)
    x = torch.ones(2, dtype=torch.float64, requires_grad=True)
    layer(x).sum().backward()
    assert torch.allclose(x.grad, torch.ones(2, dtype=torch.float64))
    return True


def test_team_collectives():
    run_ranks("test_primitives", "body_team_collectives", 4)


# ---------------------------------------------------------------- repartition
def body_repartition(rank, world, P_x_ranks, P_x_shape, P_y_ranks, P_y_shape, gshape, balanced):
    from adjoint_test import check_adjoint_test_tight
    from distdl_b200.nn import Repartition
    from distdl_b200.utilities.slicing import compute_start_index, compute_subshape
    from distdl_b200.utilities.torch import zero_volume_tensor
    P_x, P_y = _P(P_x_ranks, P_x_shape), _P(P_y_ranks, P_y_shape)
    layer = Repartition(P_x, P_y, preserve_batch=False)
    G = torch.arange(int(np.prod(gshape)), dtype=torch.float64).reshape(gshape)
    x = zero_volume_tensor(dtype=torch.float64)
    if P_x.active:
        if balanced:
            lo = compute_start_index(P_x.shape, P_x.index, gshape)
            sh = compute_subshape(P_x.shape, P_x.index, gshape)
        else:  # last worker along dim 0 takes what the others leave (others take 1 row)
            p0 = int(P_x.shape[0])
            rows = [1] * (p0 - 1) + [gshape[0] - (p0 - 1)]
            lo = compute_start_index(P_x.shape, P_x.index, gshape)
            sh = compute_subshape(P_x.shape, P_x.index, gshape)
            lo[0] = sum(rows[: int(P_x.index[0])])
            sh[0] = rows[int(P_x.index[0])]
        x = G[tuple(slice(int(a), int(a + b)) for a, b in zip(lo, sh))].clone()
    x.requires_grad = True
    y = layer(x)
    dy = zero_volume_tensor(dtype=torch.float64)
    if P_y.active:
        lo = compute_start_index(P_y.shape, P_y.index, gshape)
        sh = compute_subshape(P_y.shape, P_y.index, gshape)
        want = G[tuple(slice(int(a), int(a + b)) for a, b in zip(lo, sh))]
        assert torch.equal(y.detach(), want), f"rank {rank}: {y} vs {want}"
        dy = torch.randn(*want.shape, dtype=torch.float64)
    y.backward(dy)
    check_adjoint_test_tight(x.detach(), x.grad, y.detach(), dy)
    if P_x == P_y:
        assert all(p in ("self", None) for _, _, p in layer.P_x_to_y_overlaps) or layer.identity
    return True


REPART_CASES = [
    ([0, 1, 2, 3], [4, 1], [0, 1, 2, 3], [2, 2], [7, 5], True),     # overlapping (the 4x1 -> 2x2 example)
    ([0, 1], [1, 2], [2, 3], [2, 1], [5, 6], True),                 # disjoint
    ([0, 1], [2, 1], [3], [1, 1], [5, 4], True),                    # gather with an idle rank
    ([0], [1, 1], [0, 1, 2, 3], [2, 2], [5, 4], True),              # scatter
    ([0, 1, 2, 3], [2, 2], [0, 1, 2, 3], [2, 2], [6, 6], True),     # identity
    ([0, 1, 2], [3, 1], [0, 1, 2, 3], [2, 2], [7, 5], False),       # unbalanced input
    ([0, 1, 2, 3], [1, 4], [0, 1, 2, 3], [4, 1], [8, 8], True),     # row <-> column transpose
]


@pytest.mark.parametrize("case", REPART_CASES)
def test_repartition(case):
    run_ranks("test_primitives", "body_repartition", 4, case)


def body_repartition_errors(rank, world):
    from distdl_b200.nn import Repartition
    P_x, P_y = _P([0, 1, 2, 3], [2, 2]), _P([0, 1, 2, 3], [4])
    with pytest.raises(ValueError):
        Repartition(P_x, P_y)
    P_y = _P([0, 1, 2, 3], [1, 4])
    layer = Repartition(P_x, P_y)
    with pytest.raises(ValueError):
        layer(torch.zeros(3, 2, 2))       # tensor rank != partition rank
    P_x1, P_y1 = _P([0], [1, 1]), _P([0, 1], [1, 2])
    layer = Repartition(P_x1, P_y1)
    if rank in (0, 1):
        with pytest.raises(ValueError):
            layer(torch.zeros(3, 1) if rank == 0 else torch.zeros(0))  # size-1 dim cannot be split
    return True


def test_repartition_errors():
    run_ranks("test_primitives", "body_repartition_errors", 4)


# ------------------------------------------------- topology matrix on six workers
def body_gather_scatter_matrix(rank, world):
    """AllGather / ReduceScatter / AllSumReduce on 2 x 3 and 1 x 2 x 3 grids, along every
    dimension, with ``axes_keep`` as well as the explicit axes, even and uneven extents: shapes,
    values against the assembled global tensor, and the adjoint identity."""
    from adjoint_test import check_adjoint_test_tight
    from distdl_b200.nn import AllGather, AllSumReduce, ReduceScatter
    from distdl_b200.utilities.slicing import compute_start_index, compute_subshape
    for pshape, gshape in (([2, 3], [4, 9]), ([2, 3], [5, 7]), ([1, 2, 3], [2, 6, 7])):
        P = _P(list(range(6)), pshape)
        dim = len(pshape)
        torch.manual_seed(7)                       # the same global tensor on every worker
        G = torch.randn(*gshape, dtype=torch.float64)
        lo, sh = compute_start_index(P.shape, P.index, gshape), compute_subshape(P.shape, P.index, gshape)
        local = G[tuple(slice(int(a), int(a + b)) for a, b in zip(lo, sh))].clone()
        for axis in range(dim):
            keep = tuple(a for a in range(dim) if a != axis)
            for kw in (dict(axes_all_gather=(axis,)), dict(axes_keep=keep)):
                x = local.clone().requires_grad_()
                y = AllGather(P, **kw)(x)
                sl = [slice(int(a), int(a + b)) for a, b in zip(lo, sh)]
                sl[axis] = slice(None)
                assert torch.equal(y.detach(), G[tuple(sl)]), (pshape, gshape, axis)
                dy = torch.randn_like(y)
                y.backward(dy)
                check_adjoint_test_tight(x.detach(), x.grad, y.detach(), dy)
            # reduce-scatter of the gathered slab: every worker of the team adds the same slab, so
            # the result is team size times the own block
            for kw in (dict(axes_reduce_scatter=(axis,)), dict(axes_keep=keep)):
                sl = [slice(int(a), int(a + b)) for a, b in zip(lo, sh)]
                sl[axis] = slice(None)
                x = G[tuple(sl)].clone().requires_grad_()
                y = ReduceScatter(P, **kw)(x)
                assert torch.allclose(y.detach(), local * pshape[axis]), (pshape, gshape, axis)
                dy = torch.randn_like(y)
                y.backward(dy)
                check_adjoint_test_tight(x.detach(), x.grad, y.detach(), dy)
            for kw in (dict(axes_reduce=(axis,)), dict(axes_keep=keep)):
                x = torch.full((3, 2), float(rank + 1), dtype=torch.float64, requires_grad=True)
                y = AllSumReduce(P, **kw)(x)
                team = [r for r in range(6) if all(
                    a == axis or P.cartesian_index(r)[a] == P.index[a] for a in range(dim))]
                assert torch.allclose(y.detach(), torch.full((3, 2), float(sum(r + 1 for r in team)),
                                                             dtype=torch.float64)), (pshape, axis, team)
                dy = torch.randn_like(y)
                y.backward(dy)
                check_adjoint_test_tight(x.detach(), x.grad, y.detach(), dy)
    return True


def test_gather_scatter_allreduce_topology_matrix():
    run_ranks("test_primitives", "body_gather_scatter_matrix", 6, timeout=300)


# ------------------------------------------- partitions that once deadlocked; dtypes
def body_send_recv_pairs(rank, world, P_x_ranks, P_x_shape, P_w_ranks, P_w_shape):
    """Source partition in the middle of the rank range, destination over all ranks: the order in
    which the send / receive teams are created must not deadlock
    (``tests/primitives/test_broadcast.py:212-285`` of the reference), and the broadcast works."""
    from distdl_b200.nn import Broadcast
    from distdl_b200.utilities.torch import zero_volume_tensor
    P_x, P_w = _P(P_x_ranks, P_x_shape), _P(P_w_ranks, P_w_shape)
    layer = Broadcast(P_x, P_w, preserve_batch=False)
    x = torch.full((2, 3), float(P_x.rank + 1)) if P_x.active else zero_volume_tensor()
    y = layer(x)
    assert tuple(y.shape) == (2, 3)
    # the source of a destination worker is the source worker with the same index in the matching dims
    src_index = [i if int(p) > 1 else 0 for i, p in zip(P_w.index, [1] * (P_w.dim - P_x.dim) + list(P_x.shape))]
    want = int(np.ravel_multi_index(src_index[P_w.dim - P_x.dim:], [int(p) for p in P_x.shape])) + 1
    assert (y == want).all(), (rank, y, want)
    return True


def test_potentially_deadlocked_send_recv_pairs():
    run_ranks("test_primitives", "body_send_recv_pairs", 4, ([1, 2], [1, 2], [0, 1, 2, 3], [2, 2]))
    run_ranks("test_primitives", "body_send_recv_pairs", 8, ([2, 3, 4, 5], [1, 2, 2], list(range(8)), [2, 2, 2]),
              timeout=240)


def body_dtypes(rank, world):
    """Broadcast, SumReduce, Repartition, AllGather and HaloExchange keep the dtype of their input
    (float32, float64, bfloat16 with gradients; int32 and int64 forward only)."""
    from distdl_b200.nn import AllGather, Broadcast, HaloExchange, Repartition, SumReduce
    from distdl_b200.utilities.torch import zero_volume_tensor
    P_one, P_all, P_col = _P([0], [1, 1]), _P([0, 1, 2, 3], [2, 2]), _P([0, 1, 2, 3], [1, 4])
    for dtype, backward in ((torch.float32, True), (torch.float64, True), (torch.bfloat16, True),
                            (torch.int32, False), (torch.int64, False)):
        def data(shape, active=True):
            if not active:
                return zero_volume_tensor(dtype=dtype)
            return (10 * torch.randn(*shape)).to(dtype)
        for make, P_in, P_out, shape in ((lambda: Broadcast(P_one, P_all, preserve_batch=False), P_one, P_all, (3, 4)),
                                         (lambda: SumReduce(P_all, P_one, preserve_batch=False), P_all, P_one, (3, 4)),
                                         (lambda: Repartition(P_all, P_col, preserve_batch=False), P_all, P_col, (2, 6)),
                                         (lambda: AllGather(P_all, axes_all_gather=(1,)), P_all, P_all, (2, 3))):
            x = data(shape, P_in.active)
            x.requires_grad = backward
            y = make()(x)
            if P_out.active:
                assert y.dtype == dtype, (dtype, y.dtype)
            if backward:
                y.backward(torch.ones_like(y))
                if P_in.active:
                    assert x.grad.dtype == dtype and x.grad.shape == x.shape
        P_h = _P([0, 1, 2, 3], [1, 4])
        left, right = int(P_h.index[1] > 0), int(P_h.index[1] < 3)
        halo = np.array([[0, 0], [left, right]])
        x = data((2, 3 + left + right))
        y = HaloExchange(P_h, halo, halo, halo)(x)
        assert y.dtype == dtype and y.shape == x.shape
    return True


def test_primitives_keep_dtypes():
    run_ranks("test_primitives", "body_dtypes", 4, timeout=240)


# -------------------------------------------------------------- halo exchange
def body_halo(rank, world):
    from adjoint_test import check_adjoint_test_tight
    from distdl_b200.nn import HaloExchange
    P = _P([0, 1, 2, 3], [1, 1, 2, 2])
    halo = np.array([[0, 0], [0, 0], [1, 1], [1, 1]])
    # ghost regions only exist towards a neighbour
    idx = P.index
    halo_local = halo.copy()
    for d in (2, 3):
        if idx[d] == 0:
            halo_local[d][0] = 0
        if idx[d] == P.shape[d] - 1:
            halo_local[d][1] = 0
    layer = HaloExchange(P, halo_local, halo_local, halo_local)
    bulk = 3
    shape = [1, 1] + [bulk + halo_local[d][0] + halo_local[d][1] for d in (2, 3)]
    x = torch.zeros(*shape, dtype=torch.float64)
    inner = tuple(slice(int(halo_local[d][0]), int(shape[d] - halo_local[d][1])) for d in range(4))
    x[inner] = float(rank + 1)
    x.requires_grad = True
    y = layer(x)
    yd = y.detach()
    # every ghost cell now holds the neighbour's value, corners included
    neigh = {0: {"r": 2, "d": 3, "c": 4}, 1: {"l": 1, "d": 4, "c": 3}, 2: {"r": 4, "u": 1, "c": 2},
             3: {"l": 3, "u": 2, "c": 1}}[rank]
    if rank == 0:
        assert (yd[0, 0, :3, 3] == 2).all() and (yd[0, 0, 3, :3] == 3).all() and yd[0, 0, 3, 3] == 4
    if rank == 3:
        assert (yd[0, 0, 1:, 0] == 3).all() and (yd[0, 0, 0, 1:] == 2).all() and yd[0, 0, 0, 0] == 1
    dy = torch.randn(*shape, dtype=torch.float64)
    x2 = torch.randn(*shape, dtype=torch.float64, requires_grad=True)
    y2 = layer(x2)
    y2.backward(dy)
    check_adjoint_test_tight(x2.detach(), x2.grad, y2.detach(), dy)
    # accumulate mode: the same exchange run backwards (ghosts are added to the neighbours' bulk and
    # cleared); its adjoint is the plain exchange, and it is the transpose of the operator above
    acc = HaloExchange(P, halo_local, halo_local, halo_local, accumulate=True)
    x3 = torch.randn(*shape, dtype=torch.float64, requires_grad=True)
    y3 = acc(x3)
    y3.backward(dy)
    check_adjoint_test_tight(x3.detach(), x3.grad, y3.detach(), dy)
    assert torch.equal(x3.grad, layer(dy.clone()).detach())
    ghost = torch.ones(*shape, dtype=torch.bool)
    ghost[inner] = False
    assert (y3.detach()[ghost] == 0).all()
    return True


def test_halo_exchange():
    run_ranks("test_primitives", "body_halo", 4)


def body_halo_generic(rank, world, grid, width, bulk):
    """Any Cartesian grid: every worker holds its block of a global tensor plus ``width`` ghost layers
    towards each existing neighbour; after the exchange the ghosts (edges AND corners) equal the
    global tensor, and the exchange passes the adjoint test."""
    from adjoint_test import check_adjoint_test_tight
    from distdl_b200.nn import HaloExchange
    P = _P(list(range(world)), grid)
    dims = len(grid)
    idx = [int(i) for i in P.index]
    n = [g * b for g, b in zip(grid, bulk)]
    G = torch.arange(int(np.prod(n)), dtype=torch.float64).reshape(n)
    halo = np.zeros((dims, 2), dtype=int)
    for d in range(dims):
        if grid[d] > 1:
            halo[d][0] = width if idx[d] > 0 else 0
            halo[d][1] = width if idx[d] < grid[d] - 1 else 0
    window = tuple(slice(idx[d] * bulk[d] - int(halo[d][0]), (idx[d] + 1) * bulk[d] + int(halo[d][1]))
                   for d in range(dims))
    want = G[window].clone()
    x = torch.zeros_like(want)
    inner = tuple(slice(int(halo[d][0]), int(halo[d][0]) + bulk[d]) for d in range(dims))
    x[inner] = want[inner]
    layer = HaloExchange(P, halo, halo, halo)
    x.requires_grad = True
    y = layer(x)
    assert torch.equal(y.detach(), want), (rank, (y.detach() - want).abs().max())
    dy = torch.randn_like(y)
    x2 = torch.randn_like(want).requires_grad_()
    y2 = layer(x2)
    y2.backward(dy)
    check_adjoint_test_tight(x2.detach(), x2.grad, y2.detach(), dy)
    return True


@pytest.mark.parametrize("grid,width,bulk", [([3], 2, [5]), ([2, 3], 1, [3, 4]), ([1, 2, 1, 2], 2, [2, 3, 2, 4]),
                                             ([2, 2, 2], 1, [2, 3, 2])])
def test_halo_exchange_on_any_grid(grid, width, bulk):
    run_ranks("test_primitives", "body_halo_generic", int(np.prod(grid)), (grid, width, bulk))


def body_staging_buffers_carry_the_messages(rank, world):
    """The views that HaloExchange and Repartition obtain from their buffer manager are what travels:
    after a call, a send view holds the packed face / overlap and a receive view what arrived."""
    import distdl_b200
    from distdl_b200.nn import HaloExchange, Repartition
    be = distdl_b200.backends.backend
    # 1-D chain of 2 workers, halo width 1 towards the neighbour
    P = _P([0, 1], [1, 1, 2])
    hl, hr = int(rank > 0), int(rank < 1)
    halo = np.array([[0, 0], [0, 0], [hl, hr]])
    manager = be.BufferManager()
    layer = HaloExchange(P, halo, halo, halo, buffer_manager=manager)
    x = torch.zeros(2, 3, 4 + hl + hr, dtype=torch.float64)
    x[:, :, hl:hl + 4] = torch.arange(4, dtype=torch.float64) + 10 * (rank + 1)
    y = layer(x)
    views = layer.buffers[2]                      # [left send, left recv, right send, right recv]
    if rank == 0:
        assert views[2] is not None and torch.equal(views[2], x[:, :, 3:4])        # my last bulk column went right
        assert torch.equal(views[3], y[:, :, 4:5]) and (views[3] == 20).all()      # the neighbour's first column arrived
    else:
        assert torch.equal(views[0], x[:, :, 1:2]) and (views[1] == 13).all()
    assert len(manager.buffers_map[torch.float64]) == 4
    # repartition rows -> columns of a [4, 4] tensor over 2 workers
    P_rows, P_cols = _P([0, 1], [2, 1]), _P([0, 1], [1, 2])
    rp = Repartition(P_rows, P_cols, buffer_manager=manager)
    full = torch.arange(16, dtype=torch.float64).reshape(4, 4)
    out = rp(full[2 * rank:2 * rank + 2].clone())
    assert torch.equal(out, full[:, 2 * rank:2 * rank + 2])
    other = 1 - rank
    sent = [b for b, (sl, sh, partner) in zip(rp.P_x_to_y_buffers, rp.P_x_to_y_overlaps) if b is not None]
    got = [b for b, (sl, sh, partner) in zip(rp.P_y_to_x_buffers, rp.P_y_to_x_overlaps) if b is not None]
    assert len(sent) == 1 and torch.equal(sent[0], full[2 * rank:2 * rank + 2, 2 * other:2 * other + 2])
    assert len(got) == 1 and torch.equal(got[0], full[2 * other:2 * other + 2, 2 * rank:2 * rank + 2])
    return True


def test_staging_buffers_carry_the_messages():
    run_ranks("test_primitives", "body_staging_buffers_carry_the_messages", 2)


def body_allgather_skips_adjoint_when_gradient_goes_elsewhere(rank, world):
    """A parameter whose gradient is accumulated outside of autograd (``full_grad_view``)
    yields no gradient for its gathered copy; the adjoint reduce-scatter is then skipped on
    every member alike (nothing hangs) and the parameter receives no ``.grad``; a gathered
    tensor that simply is not used still gets an exact zero gradient."""
    import distdl_b200
    from distdl_b200.nn import AllGather
    P_world = distdl_b200.backends.backend.Partition()
    P = P_world.create_partition_inclusive(range(world)).create_cartesian_topology_partition([world, 1])
    gather = AllGather(P, axes_all_gather=(0,))
    w = torch.nn.Parameter(torch.randn(3, 4))
    w.full_grad_view = torch.zeros(world * 12)           # marks "accumulated elsewhere"
    other = torch.nn.Parameter(torch.randn(3, 4))
    full = gather(w)
    full_other = gather(other)
    unused = gather(torch.nn.Parameter(torch.ones(3, 4)))
    assert full.shape == (3 * world, 4) and unused.shape == (3 * world, 4)
    (full_other.sum() * 2.0 + full.detach().sum()).backward()
    assert w.grad is None
    assert torch.allclose(other.grad, torch.full((3, 4), 2.0 * world))
    return True


def test_allgather_adjoint_skipped_without_gradient():
    run_ranks("test_primitives", "body_allgather_skips_adjoint_when_gradient_goes_elsewhere", 2, timeout=120)
