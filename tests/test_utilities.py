"""Utilities that need no process group: balanced splits, intersections, index helpers, dtype
tables, growable buffers and the halo arithmetic of sliding-window layers (golden values of a
4-worker pooling case)."""
import numpy as np
import pytest
import torch

from distdl_b200.backends.common.buffer import BufferManager, ExpandableBuffer
from distdl_b200.nn.mixins.halo_mixin import HaloMixin
from distdl_b200.nn.mixins.pooling_mixin import PoolingMixin
from distdl_b200.utilities import slicing
from distdl_b200.utilities.tensor_decomposition import (compute_subtensor_intersection_slice,
                                                        compute_subtensor_shapes_balanced,
                                                        compute_subtensor_start_indices,
                                                        compute_subtensor_stop_indices)
from distdl_b200.utilities.torch import TensorStructure, zero_volume_tensor


def test_balanced_split_rule():
    # n over P workers: n // P each, the first n % P get one more
    shapes = [int(slicing.compute_subshape([4], [i], [10])[0]) for i in range(4)]
    assert shapes == [3, 3, 2, 2]
    starts = [int(slicing.compute_start_index([4], [i], [10])[0]) for i in range(4)]
    stops = [int(slicing.compute_stop_index([4], [i], [10])[0]) for i in range(4)]
    assert starts == [0, 3, 6, 8] and stops == [3, 6, 8, 10]
    assert list(slicing.compute_subshape([2, 3], [1, 2], [7, 8])) == [3, 2]
    assert list(slicing.compute_subshape_along_axis([4], [1], [10, 5], 0)) == [3, 5]


def test_partition_intersection_and_slices():
    # rows split over 2 workers vs columns split over 2 workers of a [4, 6] tensor
    sl = slicing.compute_partition_intersection([2, 1], [0, 0], [1, 2], [0, 1], [4, 6])
    assert sl is not None
    assert list(slicing.compute_nd_slice_shape(sl)) == [2, 3]
    assert slicing.compute_nd_slice_volume(sl) == 6
    lo, hi, extent = slicing.compute_intersection(np.array([0]), np.array([2]), np.array([2]), np.array([4]))
    assert extent.tolist() == [0]                            # the ranges only touch
    lo, hi, extent = slicing.compute_intersection(np.array([0, 1]), np.array([4, 5]), np.array([2, 0]), np.array([6, 3]))
    assert lo.tolist() == [2, 1] and hi.tolist() == [4, 3] and extent.tolist() == [2, 2]
    assert slicing.assemble_slices([1, 2], [3, 5]) == (slice(1, 3, None), slice(2, 5, None))


def test_worker_layout_and_range_index():
    lay = slicing.worker_layout([2, 3])
    assert lay.shape == (2, 3) and lay.reshape(-1).tolist() == list(range(6))
    idx = list(slicing.range_index([2, 2]))
    assert [tuple(i) for i in idx] == [(0, 0), (0, 1), (1, 0), (1, 1)]


def test_tensor_decomposition_tables():
    ts = TensorStructure()
    ts.shape = torch.Size([7, 5])
    shapes = compute_subtensor_shapes_balanced(ts, [3, 2])
    assert shapes.shape[:2] == (3, 2)
    assert shapes[0, 0].tolist() == [3, 3] and shapes[2, 1].tolist() == [2, 2]
    starts = compute_subtensor_start_indices(shapes)
    stops = compute_subtensor_stop_indices(shapes)
    assert starts[1, 1].tolist() == [3, 3] and stops[2, 1].tolist() == [7, 5]
    sl = compute_subtensor_intersection_slice(starts[0, 0], stops[0, 0], np.array([2, 1]), np.array([5, 4]))
    assert sl == (slice(2, 3, None), slice(1, 3, None))


def test_zero_volume_and_structure():
    z = zero_volume_tensor()
    assert z.numel() == 0
    zb = zero_volume_tensor(5)
    assert zb.shape[0] == 5 and zb.numel() == 0
    a = TensorStructure(torch.zeros(2, 3, requires_grad=True))
    b = TensorStructure(torch.zeros(2, 3, requires_grad=True))
    assert a == b and a.shape == torch.Size([2, 3]) and a.requires_grad
    assert a != TensorStructure(torch.zeros(2, 4))


def test_expandable_buffer_keeps_contents_and_views():
    buf = ExpandableBuffer(torch.float32, 4)
    v = buf.get_view((2, 2))
    v.copy_(torch.arange(4.).view(2, 2))
    big = buf.get_view((3, 4))                     # larger than the capacity: reallocates
    assert buf.capacity >= 12 and big.shape == (3, 4)
    assert buf.get_view((2, 2)).reshape(-1).tolist() == [0., 1., 2., 3.]   # contents and view survive
    assert buf.get_view((2, 2)).data_ptr() == buf.raw_buffer.data_ptr()


def test_buffer_manager_shares_buffers_between_requests():
    bm = BufferManager()
    a = bm.request_buffers(2, torch.float32)
    b = bm.request_buffers(3, torch.float32)
    assert a[0] is b[0] and a[1] is b[1] and len(b) == 3
    c = bm.request_buffers(1, torch.float64)
    assert c[0] is not a[0] and c[0].dtype == torch.float64


class _Pool(HaloMixin, PoolingMixin):
    pass


@pytest.mark.parametrize("index,halo,send,needed", [
    (0, [[0, 0], [0, 0], [0, 1]], [[0, 0], [0, 0], [0, 0]], [[0, 1], [0, 1], [0, 4]]),
    (1, [[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [1, 0]], [[0, 1], [0, 1], [1, 3]]),
    (2, [[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [0, 0]], [[0, 1], [0, 1], [0, 2]]),
    (3, [[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [0, 0]], [[0, 1], [0, 1], [0, 2]])])
def test_halo_arithmetic_of_strided_pooling(index, halo, send, needed):
    # a length-10 signal over 4 workers (3, 3, 2, 2), window 2, stride 2: worker 0's last
    # window needs one entry of worker 1, whose own first entry is then not needed locally
    layer = _Pool()
    h, r, s, n = layer._compute_exchange_info(np.array([1, 1, 10]), np.array([2]), np.array([2]), np.array([0]),
                                              np.array([1]), True, [1, 1, 4], [0, 0, index])
    assert np.array_equal(h, np.array(halo))
    assert np.array_equal(r, np.array(halo))
    assert np.array_equal(s, np.array(send))
    assert np.array_equal(n, np.array(needed))
    assert layer._compute_exchange_info(np.array([1, 1, 10]), np.array([2]), np.array([2]), np.array([0]),
                                        np.array([1]), False, [1, 1, 4], [0, 0, index]) == (None, None, None, None)


def test_dtype_tables():
    from distdl_b200.utilities import dtype as dt
    assert dt.torch_to_numpy_dtype_dict[torch.float32] == np.float32
    assert dt.numpy_to_torch_dtype_dict[np.dtype(np.float64)] == torch.float64
    assert torch.bfloat16 in dt.torch_to_intID_dtype_dict
    back = dt.intID_to_torch_dtype_dict[dt.torch_to_intID_dtype_dict[torch.bfloat16]]
    assert back == torch.bfloat16


def test_zero_volume_corrector():
    """A worker without a loss value gets a scalar it can call backward on; the adjoint hands a
    zero-volume gradient upstream.  A real tensor passes through unchanged."""
    from distdl_b200.functional import ZeroVolumeCorrectorFunction
    empty = zero_volume_tensor(3).requires_grad_()
    s = ZeroVolumeCorrectorFunction.apply(empty)
    assert s.shape == () and float(s.detach()) == 0.0
    s.backward()
    assert empty.grad is not None and empty.grad.numel() == 0 and empty.grad.shape[0] == 3
    x = torch.randn(2, 2, requires_grad=True)
    y = ZeroVolumeCorrectorFunction.apply(x)
    y.sum().backward()
    assert torch.equal(y, x) and torch.equal(x.grad, torch.ones(2, 2))


def body_buffer_sharing_network(rank, world):
    """A network of repartitions, a spatially partitioned convolution and a pooling layer that
    share ONE buffer manager (as in the reference's buffer-management network tests,
    ``tests/utilities/test_buffer.py:128-440``): the manager ends with no more buffers than its
    hungriest layer needs, and the result equals that of the same network with a manager per layer."""
    import distdl_b200
    from distdl_b200.nn import DistributedFeatureConv2d, DistributedMaxPool2d, Repartition
    be = distdl_b200.backends.backend
    base = be.Partition().create_partition_inclusive(range(4))
    P_a, P_b = base.create_cartesian_topology_partition([1, 1, 4, 1]), base.create_cartesian_topology_partition(
        [1, 1, 2, 2])

    def network(shared):
        mk = (lambda: shared) if shared is not None else be.BufferManager
        torch.manual_seed(0)
        return [Repartition(P_a, P_b, buffer_manager=mk()),
                DistributedFeatureConv2d(P_b, 2, 3, 3, padding=1, buffer_manager=mk()),
                DistributedMaxPool2d(P_b, 2, buffer_manager=mk()),
                Repartition(P_b, P_a, buffer_manager=mk())]

    def run(layers, x):
        for layer in layers:
            x = layer(x)
        return x
    bm = be.BufferManager()
    shared, separate = network(bm), network(None)
    if rank == 0:                                   # same kernel in both networks
        with torch.no_grad():
            separate[1].weight.copy_(shared[1].weight)
            separate[1].bias.copy_(shared[1].bias)
    torch.manual_seed(1 + rank)
    x = torch.randn(2, 2, 4, 12)
    for _ in range(2):                              # the second pass reuses every view
        y_shared, y_sep = run(shared, x), run(separate, x)
        assert torch.equal(y_shared, y_sep)
    counts = {dt: len(pool) for dt, pool in bm.buffers_map.items()}
    most = max(sum(len(pool) for pool in layer.buffer_manager.buffers_map.values()) if hasattr(layer, "buffer_manager")
               else 0 for layer in separate)
    assert sum(counts.values()) <= max(most, 4), (counts, most)
    assert sum(counts.values()) < sum(sum(len(p) for p in layer.buffer_manager.buffers_map.values())
                                      for layer in separate if hasattr(layer, "buffer_manager"))
    return True


def test_buffer_manager_shared_by_a_network_of_layers():
    from dist_harness import run_ranks
    run_ranks("test_utilities", "body_buffer_sharing_network", 4, timeout=240)


def test_metrics_sink_reports_model_flops(tmp_path):
    import json
    import time

    from distdl_b200 import models
    from distdl_b200.parallel import MetricsSink
    cfg = models.llama3_8b()
    # 6 FLOPs per matrix weight and token plus causal attention: about 48 GFLOP per token at 4096
    assert 47e9 < cfg.train_flops_per_token() < 50e9
    assert cfg.train_flops_per_token(8192) > cfg.train_flops_per_token(4096)
    moe = models.mixtral_8x7b()
    assert moe.train_flops_per_token() < 6.0 * moe.num_parameters() / 2      # two of eight experts per token
    path = tmp_path / "m.jsonl"
    sink = MetricsSink(str(path), flops_per_token=1e9, peak_tflops=1.0)
    sink.step(1, 2.0, tokens=1000)
    time.sleep(0.05)
    sink.step(2, 1.5, tokens=1000, lr=1e-3, grad_norm=0.7)
    sink.close()
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    assert rows[0]["ms_per_step"] is None and "model_tflops_per_gpu" not in rows[0]
    r = rows[1]
    assert abs(r["model_tflops_per_gpu"] - r["tokens_per_s"] * 1e9 / 1e12) < 1e-9
    assert abs(r["fraction_of_peak"] - r["model_tflops_per_gpu"]) < 1e-12 and r["grad_norm"] == 0.7


def test_buffer_allocators_assign_views_per_message():
    """Repartition: one buffer per message that leaves or enters (none for "self" / empty overlaps),
    sends first; halo exchange: four buffers re-viewed per dimension."""
    from distdl_b200.backends.common.buffer_allocator import (allocate_halo_exchange_buffers,
                                                              allocate_repartition_buffers)
    bm = BufferManager()
    sl = (slice(0, 2), slice(0, 3))
    x_to_y = [(sl, (2, 3), 1), (sl, (2, 3), "self"), (None, None, None), (sl, (4, 1), 3)]
    y_to_x = [(sl, (5,), 2), (sl, (2, 3), "self")]
    send, recv = allocate_repartition_buffers(bm, x_to_y, y_to_x, torch.float32)
    assert [None if v is None else tuple(v.shape) for v in send] == [(2, 3), None, None, (4, 1)]
    assert [None if v is None else tuple(v.shape) for v in recv] == [(5,), None]
    assert len(bm.buffers_map[torch.float32]) == 3                 # two sends + one receive
    assert send[0].data_ptr() != send[3].data_ptr() != recv[0].data_ptr()
    # a second layer with smaller messages reuses the same three buffers
    send2, _ = allocate_repartition_buffers(bm, [(sl, (1, 2), 1)], [], torch.float32)
    assert len(bm.buffers_map[torch.float32]) == 3 and send2[0].data_ptr() == send[0].data_ptr()
    # halo exchange on a [6, 8] tensor with width-1 halos in both dimensions
    def s(a, b):
        return slice(a, b)
    slices = [((s(1, 2), s(1, 7)), (s(0, 1), s(1, 7)), (s(4, 5), s(1, 7)), (s(5, 6), s(1, 7))),
              ((s(0, 6), s(1, 2)), (s(0, 6), s(0, 1)), (s(0, 6), s(6, 7)), (s(0, 6), s(7, 8)))]
    widths = np.array([[1, 1], [1, 0]])                            # nothing moves to / from the right in dim 1
    views = allocate_halo_exchange_buffers(bm, slices, widths, widths, torch.float32)
    assert [tuple(v.shape) for v in views[0]] == [(1, 6)] * 4
    assert tuple(views[1][0].shape) == (6, 1) and views[1][2] is None and views[1][3] is None
    assert len(bm.buffers_map[torch.float32]) == 4                 # the manager grew to the halo layer's four


@pytest.mark.parametrize("nd", [1, 2, 3])
@pytest.mark.parametrize("mode,ac", [("nearest", False), ("linear", False), ("linear", True)])
def test_interpolate_function_cpu_adjoint_and_values(nd, mode, ac):
    """The native interpolation on CPU tensors, fp64: equals torch's interpolation on whole tensors,
    a sub-slab in global coordinates equals the matching slice of the whole result, and the backward
    pass is the exact adjoint (dot-product test)."""
    from distdl_b200.functional.interpolate import InterpolateFunction
    torch.manual_seed(nd)
    n_in, n_out = [5, 6, 4][:nd], [11, 9, 10][:nd]
    x = torch.randn(2, 3, *n_in, dtype=torch.float64, requires_grad=True)
    zeros = [0] * nd
    y = InterpolateFunction.apply(x, zeros, n_in, n_in, zeros, n_out, n_out, None, mode, ac)
    tmode = {1: "linear", 2: "bilinear", 3: "trilinear"}[nd] if mode == "linear" else "nearest"
    want = torch.nn.functional.interpolate(x.detach(), size=n_out, mode=tmode,
                                           **({} if mode == "nearest" else {"align_corners": ac}))
    assert torch.allclose(y, want, atol=1e-12), (y - want).abs().max()
    dy = torch.randn_like(y)
    y.backward(dy)
    lhs, rhs = (y.detach() * dy).sum(), (x.detach() * x.grad).sum()
    assert abs(lhs - rhs) < 1e-10 * max(1.0, abs(lhs)), (lhs, rhs)
    # output slab [3, 8) of the first spatial dimension, computed from the whole input
    lo, hi = 3, 8
    y_lo, y_hi = [lo] + zeros[1:], [hi] + n_out[1:]
    part = InterpolateFunction.apply(x.detach(), zeros, n_in, n_in, y_lo, y_hi, n_out, None, mode, ac)
    assert torch.allclose(part, want[:, :, lo:hi], atol=1e-12)


def test_conv_mixin_input_ranges():
    from distdl_b200.nn.mixins.conv_mixin import ConvMixin
    m = ConvMixin()
    # kernel 3, stride 2, padding 1, dilation 2: output 4 reads inputs 7 .. 11
    assert m._compute_min_input_range(4, 3, 2, 1, 2) == 7 and m._compute_max_input_range(4, 3, 2, 1, 2) == 11
    assert m._compute_min_input_range(0, 3, 1, 1, 1) == -1 and m._compute_max_input_range(0, 3, 1, 1, 1) == 1


@pytest.mark.parametrize("mode,ac", [("nearest", False), ("linear", False), ("linear", True)])
@pytest.mark.parametrize("n_in,n_out", [(16, 32), (10, 25), (12, 7)])
def test_interpolate_mixin_needed_range_covers_what_torch_reads(mode, ac, n_in, n_out):
    """For every output slab, the input range that the mixin asks for is exactly wide enough: interpolating
    the slab from that range alone (in global coordinates) reproduces torch's result on the whole tensor."""
    from distdl_b200.functional.interpolate import InterpolateFunction
    from distdl_b200.nn.mixins.interpolate_mixin import InterpolateMixin
    m = InterpolateMixin()
    torch.manual_seed(0)
    x = torch.randn(1, 2, n_in, dtype=torch.float64)
    want = torch.nn.functional.interpolate(x, size=n_out, mode=mode, **({} if mode == "nearest" else
                                                                        {"align_corners": ac}))
    for y_lo, y_hi in ((0, n_out // 3), (n_out // 3, 2 * n_out // 3), (2 * n_out // 3, n_out)):
        lo, hi = m._compute_needed_range([y_lo], [y_hi], [n_in], [n_out], [None], mode, ac)
        lo, hi = int(lo[0]), int(hi[0])
        assert 0 <= lo < hi <= n_in
        part = InterpolateFunction.apply(x[:, :, lo:hi].contiguous(), [lo], [hi], [n_in], [y_lo], [y_hi], [n_out],
                                         None, mode, ac)
        assert torch.allclose(part, want[:, :, y_lo:y_hi], atol=1e-12), (mode, ac, y_lo, y_hi, lo, hi)
