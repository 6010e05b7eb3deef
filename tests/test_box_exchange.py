"""The box exchange without a GPU: the geometry that the host computes (collapsed boxes, copy
units), the kernel's index arithmetic (compiled for the host as well) against PyTorch slicing,
the way plans are cut into launches, and whole halo exchanges / repartitions on CPU ranks with
the plan executed by ``BoxPlan.run_on_host`` against the slicing formulation."""

import pytest
import torch

from dist_harness import run_ranks


def test_collapse_merges_contiguous_dimensions_and_picks_the_copy_unit():
    from distdl_b200.parallel.box_exchange import collapse
    # a whole contiguous tensor is one run
    assert collapse([4, 6, 8], [48, 8, 1], 4, True) == ([1, 1, 1, 4 * 6 * 8 * 4 // 16], [0, 0, 0], 16)
    # a face of width 1 in the last dimension: element-wise, one outer direction per sliced dim
    n, s, unit = collapse([4, 6, 1], [48, 8, 1], 4, True)
    assert unit == 4 and n == [1, 1, 24, 1] and s == [0, 0, 32]
    # inner run of 8 floats = 32 bytes, but the start is not 16-byte aligned
    assert collapse([4, 8], [16, 1], 4, False)[2] == 4
    assert collapse([4, 8], [16, 1], 4, True) == ([1, 1, 4, 2], [0, 0, 64], 16)
    # five genuinely strided dimensions do not fit
    assert collapse([2, 2, 2, 2, 2], [1000, 100, 20, 6, 2], 4, True) is None


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.int64, torch.uint8, torch.bfloat16])
def test_host_index_arithmetic_matches_slicing(dtype):
    from distdl_b200.parallel.box_exchange import host_copy
    gen = torch.Generator().manual_seed(0)
    shape = (3, 4, 9, 8)
    base = (torch.randn(shape, generator=gen) * 50).to(dtype)
    boxes = [(slice(0, 3), slice(0, 4), slice(0, 9), slice(0, 8)), (slice(1, 3), slice(0, 4), slice(2, 3), slice(0, 8)),
             (slice(0, 3), slice(1, 2), slice(0, 9), slice(7, 8)), (slice(2, 3), slice(1, 4), slice(3, 8), slice(4, 8)),
             (slice(0, 3), slice(0, 4), slice(4, 9), slice(0, 4))]
    for sl in boxes:
        x = base.clone()
        want = x[sl].contiguous()
        flat = torch.zeros(want.numel() * want.element_size(), dtype=torch.uint8)
        assert host_copy("send", x, sl, flat)
        assert torch.equal(flat.view(dtype).view(want.shape), want)
        y = torch.zeros_like(base)
        assert host_copy("recv", y, sl, flat)
        assert torch.equal(y[sl], want) and y.ne(0).sum() == want.ne(0).sum()
        # pack with clearing; unpack with addition (the adjoint of the halo exchange)
        flat2 = torch.zeros_like(flat)
        assert host_copy("send", x, sl, flat2, clear=True)
        assert torch.equal(flat2, flat) and x[sl].ne(0).sum() == 0
        if dtype in (torch.float32, torch.float64):
            z = base.clone()
            assert host_copy("recv", z, sl, flat, add=True)
            assert torch.equal(z[sl], base[sl] * 2)
    # a transposed (non-contiguous) view
    xt = base.clone().permute(0, 2, 1, 3)
    sl = (slice(0, 2), slice(1, 5), slice(0, 4), slice(2, 6))
    want = xt[sl].contiguous()
    flat = torch.zeros(want.numel() * want.element_size(), dtype=torch.uint8)
    assert host_copy("send", xt, sl, flat)
    assert torch.equal(flat.view(dtype).view(want.shape), want)


def test_plans_are_cut_into_launches_where_the_kernel_cannot_take_a_box():
    from distdl_b200.parallel.box_exchange import BoxPlan, _limits, pieces_of
    _max_items, chunk, piece = _limits()
    x = torch.zeros(4, 6, 8, 10)
    full = (slice(0, 4), slice(0, 6), slice(0, 8), slice(0, 10))
    face = (slice(0, 4), slice(0, 6), slice(0, 8), slice(0, 1))
    plan = BoxPlan([[("send", 1, "x", face, False), ("recv", 1, "x", face, False)],
                    [("send", 2, "x", full, True), ("recv", 2, "x", full, True)]])
    launches = plan._compile({"x": BoxPlan._meta(x)})
    assert len(launches) == 1
    items, phase_pieces, pre, post = launches[0]
    assert [it[-1] for it in items] == [0, 0, 1, 1] and not pre and not post
    assert phase_pieces == [2 * pieces_of(4 * 6 * 8 * 4, chunk, piece[4]), 2 * pieces_of(x.numel() * 4, chunk, piece[16])]
    # an integer tensor cannot be added by the kernel: that phase runs through a temporary, alone in its launch
    xi = torch.zeros(4, 6, dtype=torch.int32)
    plan = BoxPlan([[("send", 1, "x", None, False)], [("recv", 1, "x", None, True)], [("send", 1, "x", None, False)]])
    launches = plan._compile({"x": BoxPlan._meta(xi)})
    assert len(launches) == 3 and launches[1][3] and launches[1][3][0][0] == "tmp_recv"
    # a message larger than a chunk advances the progress counter by all its pieces
    assert pieces_of(chunk + 1, chunk, piece[16]) == chunk // piece[16] + 1


class _HostBoxPlan:
    def __init__(self, plan, transport, team):
        self.plan, self.transport, self.team = plan, transport, team

    def run(self, **tensors):
        self.plan.run_on_host(self.transport, self.team, **tensors)


def _with_host_box_plans(transport_cls):
    from distdl_b200.parallel.box_exchange import BoxPlan

    class T(transport_cls):
        box_plans_on_host = True

        def box_plan(self, phases, team):
            return _HostBoxPlan(BoxPlan(phases), self, team)
    return T


def body_halo_and_repartition(rank, world):
    """Halo exchange (forward and adjoint, 3-D tensor dims with corners) and repartitions between several
    grids: the plan form against the slicing form, same inputs, on 4 CPU ranks."""
    import numpy as np

    import distdl_b200
    import distdl_b200.nn as dnn
    from distdl_b200.backends.common.functional import halo_exchange as hx
    from distdl_b200.backends.common.functional import repartition as rp
    from distdl_b200.backends.common.transport import P2PTransport
    be = distdl_b200.backends.backend
    base = be.Partition().create_partition_inclusive(range(world))
    plain = P2PTransport()
    boxed = _with_host_box_plans(P2PTransport)()
    for dtype in (torch.float32, torch.float64, torch.int64):
        P_x = base.create_cartesian_topology_partition([1, 1, 2, 2])
        halo = np.array([[0, 0], [0, 0], [2, 2], [1, 1]])
        idx = P_x.index
        for d in (2, 3):
            if idx[d] == 0:
                halo[d][0] = 0
            if idx[d] == P_x.shape[d] - 1:
                halo[d][1] = 0
        layer = dnn.HaloExchange(P_x, halo, halo, halo)
        shape = [2, 3] + [5 + halo[d][0] + halo[d][1] for d in (2, 3)]
        torch.manual_seed(10 + rank)
        x = (torch.randn(*shape) * 20).to(dtype)
        layer._distdl_module_setup((x,))
        for fn in (hx.fill_ghosts, hx.fold_ghosts):
            want = fn(plain, x, P_x, layer.slices, layer.neighbor_ranks)
            got = fn(boxed, x, P_x, layer.slices, layer.neighbor_ranks)
            assert torch.equal(want, got), (fn.__name__, dtype, (want - got).abs().max())
    # repartitions: row blocks -> column blocks, a 2 x 2 grid -> one worker, and back
    for shape_x, shape_y in (([4, 1], [1, 4]), ([2, 2], [1, 1]), ([1, 1], [2, 2]), ([2, 2], [4, 1])):
        nx, ny = int(np.prod(shape_x)), int(np.prod(shape_y))
        P_x = base.create_partition_inclusive(range(nx)).create_cartesian_topology_partition(shape_x)
        P_y = base.create_partition_inclusive(range(world - ny, world)).create_cartesian_topology_partition(shape_y)
        layer = dnn.Repartition(P_x, P_y, preserve_batch=False)
        torch.manual_seed(3)
        full = torch.randn(10, 13)
        if P_x.active:
            from distdl_b200.utilities.slicing import compute_start_index, compute_subshape
            lo = compute_start_index(P_x.shape, P_x.index, full.shape)
            n = compute_subshape(P_x.shape, P_x.index, full.shape)
            x = full[lo[0]:lo[0] + n[0], lo[1]:lo[1] + n[1]].clone()
        else:
            from distdl_b200.utilities.torch import zero_volume_tensor
            x = zero_volume_tensor()
        layer._distdl_module_setup((x,))
        sends = layer.P_x_to_y_overlaps if P_x.active else []
        recvs = layer.P_y_to_x_overlaps if P_y.active else []
        out_shape = layer.output_tensor_structure.shape if P_y.active else None
        team = list(layer.P_union.ranks)
        want = rp._move(plain, x, out_shape, torch.float32, sends, recvs, x.device, team)
        got = rp._move(boxed, x, out_shape, torch.float32, sends, recvs, x.device, team)
        assert (want is None) == (got is None)
        if want is not None:
            assert torch.equal(want, got), (shape_x, shape_y)
            lo = compute_start_index(P_y.shape, P_y.index, full.shape) if P_y.active else None
            n = compute_subshape(P_y.shape, P_y.index, full.shape)
            assert torch.equal(got, full[lo[0]:lo[0] + n[0], lo[1]:lo[1] + n[1]])
    return True


def test_halo_exchange_and_repartition_through_box_plans_on_cpu_ranks():
    run_ranks("test_box_exchange", "body_halo_and_repartition", 4, timeout=180)


def test_bounds_checking_build_compiles_and_reports_itself():
    """`python -m distdl_b200._build --debug` gives a second library in which the box-exchange kernel
    checks every computed address against the tensor's storage (violations are recorded in the
    status record and the access is skipped); the regular library does not carry the checks."""
    import ctypes

    from distdl_b200 import _build
    path = _build.build(debug=True)
    assert path.endswith("libdistdl_b200_debug.so")
    assert ctypes.CDLL(path).dd_bounds_checked() == 1
    assert ctypes.CDLL(_build.build()).dd_bounds_checked() == 0
