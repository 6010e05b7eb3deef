"""Convolution, pooling, batch-norm and loss layers against serial PyTorch on
CPU ranks, plus the halo arithmetic golden values."""
import numpy as np
import torch

from dist_harness import run_ranks


def test_halo_mixin_golden_values():
    """Expected arrays for a [1,1,10] tensor, kernel 2 / stride 2 pooling, on a
    [1,1,4] partition (values as in the reference's utility test)."""
    from distdl_b200.nn.mixins import HaloMixin, PoolingMixin

    class Mock(HaloMixin, PoolingMixin):
        pass
    want = {0: ([[0, 0], [0, 0], [0, 1]], [[0, 0], [0, 0], [0, 1]], [[0, 0], [0, 0], [0, 0]], [[0, 1], [0, 1], [0, 4]]),
            1: ([[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [1, 0]], [[0, 1], [0, 1], [1, 3]]),
            2: ([[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [0, 0]], [[0, 1], [0, 1], [0, 2]]),
            3: ([[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [0, 0]], [[0, 0], [0, 0], [0, 0]], [[0, 1], [0, 1], [0, 2]])}
    for r in range(4):
        got = Mock()._compute_exchange_info(np.array([1, 1, 10]), np.array([2]), np.array([2]), np.array([0]),
                                            np.array([1]), True, [1, 1, 4], [0, 0, r])
        for g, w in zip(got, want[r]):
            assert np.array_equal(g, np.array(w)), (r, g, w)
    assert Mock()._compute_exchange_info(np.array([1, 1, 10]), [2], [2], [0], [1], False, [1, 1, 4], [0, 0, 0]) == \
        (None, None, None, None)


def _cart(ranks, shape):
    import distdl_b200 as d
    return d.backends.backend.Partition().create_partition_inclusive(ranks).create_cartesian_topology_partition(shape)


def _scatter(P, x_global, rank, dim):
    from distdl_b200.nn import Repartition
    from distdl_b200.utilities.torch import zero_volume_tensor
    P_root = _cart([0], [1] * dim)
    x0 = x_global.clone().requires_grad_() if rank == 0 else zero_volume_tensor().requires_grad_()
    return x0, Repartition(P_root, P, preserve_batch=False)(x0)


def _gather(P, y, dim):
    from distdl_b200.nn import Repartition
    return Repartition(P, _cart([0], [1] * dim), preserve_batch=False)(y)


def _sync(t):
    import torch.distributed as dist
    dist.broadcast(t, src=0)
    return t


def body_feature_conv_pool(rank, world):
    from distdl_b200.nn import DistributedAvgPool2d, DistributedFeatureConv2d, DistributedMaxPool1d
    torch.manual_seed(0)
    P = _cart([0, 1, 2, 3], [1, 1, 2, 2])
    xg = _sync(torch.randn(2, 3, 11, 9))
    for (k, s, p, d) in [(3, 1, 1, 1), (3, 2, 1, 1), (2, 2, 0, 1), (3, 1, 2, 2)]:
        layer = DistributedFeatureConv2d(P, 3, 4, k, stride=s, padding=p, dilation=d)
        w = _sync(layer.weight.detach().clone() if rank == 0 else torch.empty(4, 3, k, k))
        b = _sync(layer.bias.detach().clone() if rank == 0 else torch.empty(4))
        x0, x = _scatter(P, xg, rank, 4)
        y = _gather(P, layer(x), 4)
        if rank == 0:
            xs = xg.clone().requires_grad_()
            ys = torch.nn.functional.conv2d(xs, w, b, stride=s, padding=p, dilation=d)
            assert y.shape == ys.shape, (y.shape, ys.shape, k, s, p, d)
            assert torch.allclose(y, ys, atol=1e-5), (k, s, p, d)
            g = torch.randn_like(ys)
            ys.backward(g)
            y.backward(g)
            assert torch.allclose(x0.grad, xs.grad, atol=1e-5)
            assert torch.allclose(layer.weight.grad, torch.autograd.grad(
                torch.nn.functional.conv2d(xg, w.requires_grad_(), b, stride=s, padding=p, dilation=d), w, g)[0],
                atol=1e-4)
        else:
            y.backward(torch.zeros_like(y))
    pool = DistributedAvgPool2d(P, 2, stride=2)
    x0, x = _scatter(P, xg, rank, 4)
    y = _gather(P, pool(x), 4)
    if rank == 0:
        assert torch.allclose(y, torch.nn.functional.avg_pool2d(xg, 2, 2), atol=1e-6)
    P1 = _cart([0, 1, 2, 3], [1, 1, 4])
    x1 = _sync(torch.randn(2, 3, 10))
    mp = DistributedMaxPool1d(P1, 3, stride=2, padding=1)
    _, x = _scatter(P1, x1, rank, 3)
    y = _gather(P1, mp(x), 3)
    if rank == 0:
        assert torch.allclose(y, torch.nn.functional.max_pool1d(x1, 3, 2, 1))
    return True


def test_feature_conv_and_pooling_vs_serial():
    run_ranks("test_layers_conv", "body_feature_conv_pool", 4, timeout=300)


def body_channel_convs(rank, world):
    from distdl_b200.nn import (DistributedChannelAllGatherConv1d, DistributedChannelConv2d, DistributedConv2d,
                                DistributedChannelReduceScatterConv1d, DistributedGeneralConv1d)
    import torch.distributed as dist
    torch.manual_seed(0)
    # --- 2-D channel conv: P_x [1,2,1,1], P_y [1,2,1,1], P_w [2,2,1,1]
    P_x, P_y, P_w = _cart([0, 1], [1, 2, 1, 1]), _cart([0, 1], [1, 2, 1, 1]), _cart([0, 1, 2, 3], [2, 2, 1, 1])
    layer = DistributedConv2d(P_x, P_y, P_w, in_channels=4, out_channels=6, kernel_size=3, padding=1)
    assert isinstance(layer, DistributedChannelConv2d)
    xg = _sync(torch.randn(2, 4, 5, 5))
    # assemble the serial weight from the blocks
    Wfull = torch.zeros(6, 4, 3, 3)
    bfull = torch.zeros(6)
    co, ci = rank // 2, rank % 2
    Wfull[co * 3:(co + 1) * 3, ci * 2:(ci + 1) * 2] = layer.conv_layer.weight.detach()
    if ci == 0:
        bfull[co * 3:(co + 1) * 3] = layer.conv_layer.bias.detach()
    dist.all_reduce(Wfull)
    dist.all_reduce(bfull)
    _, x = _scatter(P_x, xg, rank, 4)
    y = _gather(P_y, layer(x), 4)
    if rank == 0:
        assert torch.allclose(y, torch.nn.functional.conv2d(xg, Wfull, bfull, padding=1), atol=1e-5)
    # --- channel all-gather / reduce-scatter 1-D convs on [D=2, M=2, 1]
    P = _cart([0, 1, 2, 3], [2, 2, 1])
    x1 = _sync(torch.randn(4, 6, 9))
    d, m = rank // 2, rank % 2
    ag = DistributedChannelAllGatherConv1d(P, 6, 8, 3, padding=1)
    W = torch.zeros(8, 6, 3)
    b = torch.zeros(8)
    if d == 0:
        W[m * 4:(m + 1) * 4] = ag.weight.detach()
        b[m * 4:(m + 1) * 4] = ag.bias.detach()
    dist.all_reduce(W)
    dist.all_reduce(b)
    xl = x1[d * 2:(d + 1) * 2, m * 3:(m + 1) * 3].clone()
    y = ag(xl)
    want = torch.nn.functional.conv1d(x1, W, b, padding=1)[d * 2:(d + 1) * 2, m * 4:(m + 1) * 4]
    assert torch.allclose(y, want, atol=1e-5)
    rs = DistributedChannelReduceScatterConv1d(P, 6, 8, 3, padding=1)
    W = torch.zeros(8, 6, 3)
    b = torch.zeros(8)
    if d == 0:
        W[:, m * 3:(m + 1) * 3] = rs.weight.detach()
    if rank == 0:
        b = rs.bias.detach().clone()
    dist.all_reduce(W)
    dist.all_reduce(b)
    y = rs(xl)
    want = torch.nn.functional.conv1d(x1, W, b, padding=1)[d * 2:(d + 1) * 2, m * 4:(m + 1) * 4]
    assert torch.allclose(y, want, atol=1e-5)
    y.sum().backward()
    # --- general conv: channels and space split
    P_x, P_y, P_w = _cart([0, 1], [1, 1, 2]), _cart([0, 1], [1, 1, 2]), _cart([0, 1], [1, 1, 2])
    gen = DistributedGeneralConv1d(P_x, P_y, P_w, 3, 5, 3, padding=1)
    x2 = _sync(torch.randn(2, 3, 12))
    if rank in (0, 1):
        Wg = _sync_pair(gen.weight.detach().clone() if rank == 0 else torch.empty(5, 3, 3), rank)
        bg = _sync_pair(gen.bias.detach().clone() if rank == 0 else torch.empty(5), rank)
        xl = x2[:, :, rank * 6:(rank + 1) * 6].clone()
        y = gen(xl)
        want = torch.nn.functional.conv1d(x2, Wg, bg, padding=1)[:, :, rank * 6:(rank + 1) * 6]
        assert torch.allclose(y, want, atol=1e-5)
    return True


def _sync_pair(t, rank):
    """rank 0 -> rank 1 copy inside the pair {0, 1}."""
    import torch.distributed as dist
    if rank == 0:
        dist.send(t, dst=1)
    else:
        dist.recv(t, src=0)
    return t


def test_channel_and_general_convs_vs_serial():
    run_ranks("test_layers_conv", "body_channel_convs", 4, timeout=300)


def body_batchnorm_loss(rank, world):
    from distdl_b200.nn import DistributedBatchNorm, DistributedMSELoss
    torch.manual_seed(0)
    P = _cart([0, 1, 2, 3], [2, 2, 1])
    xg = _sync(torch.randn(6, 4, 5))
    d, m = rank // 2, rank % 2
    xl = xg[d * 3:(d + 1) * 3, m * 2:(m + 1) * 2].clone().requires_grad_()
    bn = DistributedBatchNorm(P, 4)
    y = bn(xl)
    ref = torch.nn.BatchNorm1d(4)
    xs = xg.clone().requires_grad_()
    ys = ref(xs)
    assert torch.allclose(y, ys[d * 3:(d + 1) * 3, m * 2:(m + 1) * 2], atol=1e-5)
    if d == 0:
        assert torch.allclose(bn.running_var.reshape(-1), ref.running_var[m * 2:(m + 1) * 2], atol=1e-5)
    tg = _sync(torch.randn(6, 4, 5))
    crit = DistributedMSELoss(P)
    loss = crit(y, tg[d * 3:(d + 1) * 3, m * 2:(m + 1) * 2])
    loss.backward()
    ls = torch.nn.functional.mse_loss(ys, tg)
    ls.backward()
    if rank == 0:
        assert abs(loss.item() - ls.item()) < 1e-6
    assert torch.allclose(xl.grad, xs.grad[d * 3:(d + 1) * 3, m * 2:(m + 1) * 2], atol=1e-6)
    return True


def test_batchnorm_and_loss_vs_serial():
    run_ranks("test_layers_conv", "body_batchnorm_loss", 4, timeout=300)


def body_upsample(rank, world):
    from distdl_b200.nn import DistributedUpsample
    torch.manual_seed(0)
    P = _cart([0, 1, 2, 3], [1, 1, 2, 2])
    xg = _sync(torch.randn(2, 2, 9, 7))
    for kw, tkw in [(dict(scale_factor=2, mode="linear"), dict(scale_factor=2, mode="bilinear")),
                    (dict(size=(20, 11), mode="linear", align_corners=True),
                     dict(size=(20, 11), mode="bilinear", align_corners=True)),
                    (dict(scale_factor=3, mode="nearest"), dict(scale_factor=3, mode="nearest"))]:
        layer = DistributedUpsample(P, **kw)
        x0, x = _scatter(P, xg, rank, 4)
        y = _gather(P, layer(x), 4)
        if rank == 0:
            xs = xg.clone().requires_grad_()
            ys = torch.nn.functional.interpolate(xs, **tkw)
            assert y.shape == ys.shape, (y.shape, ys.shape)
            assert torch.allclose(y, ys, atol=1e-5), kw
            g = torch.randn_like(ys)
            ys.backward(g)
            y.backward(g)
            assert torch.allclose(x0.grad, xs.grad, atol=1e-5), kw
        else:
            y.backward(torch.zeros_like(y))
    return True


def test_upsample_vs_serial():
    run_ranks("test_layers_conv", "body_upsample", 4, timeout=300)


def body_losses(rank, world):
    """All six distributed losses against their torch counterparts on the full tensors (value on
    worker 0, gradients on every worker), mean and sum reductions."""
    import distdl_b200.nn as dnn
    P = _cart([0, 1, 2, 3], [2, 2])
    torch.manual_seed(0)
    cases = [
        (dnn.DistributedL1Loss, torch.nn.L1Loss, lambda t: t, lambda t: t),
        (dnn.DistributedMSELoss, torch.nn.MSELoss, lambda t: t, lambda t: t),
        (dnn.DistributedPoissonNLLLoss, torch.nn.PoissonNLLLoss, lambda t: t, lambda t: t.abs()),
        (dnn.DistributedBCELoss, torch.nn.BCELoss, torch.sigmoid, torch.sigmoid),
        (dnn.DistributedBCEWithLogitsLoss, torch.nn.BCEWithLogitsLoss, lambda t: t, torch.sigmoid),
        (dnn.DistributedKLDivLoss, torch.nn.KLDivLoss, lambda t: torch.log_softmax(t, -1),
         lambda t: torch.softmax(t, -1)),
    ]
    d, m = rank // 2, rank % 2
    sl = (slice(d * 3, (d + 1) * 3), slice(m * 4, (m + 1) * 4))
    for Dist, Ref, fx, ft in cases:
        for reduction in ("mean", "sum"):
            raw_x = _sync(torch.randn(6, 8))
            raw_t = _sync(torch.randn(6, 8))
            xs = raw_x.clone().requires_grad_()
            ref = Ref(reduction=reduction)(fx(xs), ft(raw_t))
            ref.backward()
            xl = raw_x[sl].clone().requires_grad_()
            # softmax-type transforms act on full rows: apply them on the full tensor, then cut
            if Dist is dnn.DistributedKLDivLoss:
                xin = fx(raw_x)[sl].clone().requires_grad_()
            else:
                xin = fx(xl)
            loss = Dist(P, reduction=reduction)(xin, ft(raw_t)[sl])
            loss.backward()
            if rank == 0:
                assert abs(loss.item() - ref.item()) < 1e-5 * max(1.0, abs(ref.item())), (Dist.__name__, reduction)
            if Dist is not dnn.DistributedKLDivLoss:
                assert torch.allclose(xl.grad, xs.grad[sl], atol=1e-6), (Dist.__name__, reduction)
    return True


def test_all_losses_vs_serial():
    run_ranks("test_layers_conv", "body_losses", 4, timeout=300)


def body_conv_pool_other_dims(rank, world):
    """1-D and 3-D variants, transposed feature convolutions, the selector classes, the
    DistributedTranspose alias and the sub-tensor Interpolate against serial torch."""
    import distdl_b200.nn as dnn
    torch.manual_seed(0)
    # ---- 1-D feature conv + avg pool, 3-D feature conv + max pool, through the selector
    P1 = _cart([0, 1, 2, 3], [1, 1, 4])
    x1 = _sync(torch.randn(2, 3, 21))
    conv1 = dnn.DistributedConv1d(P1, in_channels=3, out_channels=5, kernel_size=3, padding=1)
    assert isinstance(conv1, dnn.DistributedFeatureConv1d)
    w = _sync(conv1.weight.detach().clone() if rank == 0 else torch.empty(5, 3, 3))
    b = _sync(conv1.bias.detach().clone() if rank == 0 else torch.empty(5))
    _, x = _scatter(P1, x1, rank, 3)
    y = _gather(P1, conv1(x), 3)
    if rank == 0:
        assert torch.allclose(y, torch.nn.functional.conv1d(x1, w, b, padding=1), atol=1e-5)
    _, x = _scatter(P1, x1, rank, 3)
    y = _gather(P1, dnn.DistributedAvgPool1d(P1, 3, stride=3)(x), 3)
    if rank == 0:
        assert torch.allclose(y, torch.nn.functional.avg_pool1d(x1, 3, 3), atol=1e-6)
    P3 = _cart([0, 1, 2, 3], [1, 1, 2, 2, 1])
    x3 = _sync(torch.randn(1, 2, 8, 6, 5))
    conv3 = dnn.DistributedConv3d(P3, in_channels=2, out_channels=3, kernel_size=3, padding=1)
    assert isinstance(conv3, dnn.DistributedFeatureConv3d)
    w = _sync(conv3.weight.detach().clone() if rank == 0 else torch.empty(3, 2, 3, 3, 3))
    b = _sync(conv3.bias.detach().clone() if rank == 0 else torch.empty(3))
    _, x = _scatter(P3, x3, rank, 5)
    y = _gather(P3, conv3(x), 5)
    if rank == 0:
        assert torch.allclose(y, torch.nn.functional.conv3d(x3, w, b, padding=1), atol=1e-5)
    for Pool, fn in ((dnn.DistributedMaxPool3d, torch.nn.functional.max_pool3d),
                     (dnn.DistributedAvgPool3d, torch.nn.functional.avg_pool3d)):
        _, x = _scatter(P3, x3, rank, 5)
        y = _gather(P3, Pool(P3, 2, stride=2)(x), 5)
        if rank == 0:
            assert torch.allclose(y, fn(x3, 2, 2), atol=1e-6), Pool.__name__
    P2 = _cart([0, 1, 2, 3], [1, 1, 2, 2])
    x2 = _sync(torch.randn(2, 3, 10, 8))
    _, x = _scatter(P2, x2, rank, 4)
    y = _gather(P2, dnn.DistributedMaxPool2d(P2, 2, stride=2)(x), 4)
    if rank == 0:
        assert torch.allclose(y, torch.nn.functional.max_pool2d(x2, 2, 2))
    # ---- the alias and the selector's other branches
    assert issubclass(dnn.DistributedTranspose, dnn.Repartition)
    Pc_x, Pc_y, Pc_w = _cart([0, 1], [1, 2, 1]), _cart([0, 1], [1, 2, 1]), _cart([0, 1, 2, 3], [2, 2, 1])
    assert isinstance(dnn.DistributedConv1d(Pc_x, Pc_y, Pc_w, in_channels=4, out_channels=4, kernel_size=1),
                      dnn.DistributedChannelConv1d)
    return True


def test_other_dimensions_selector_and_alias():
    run_ranks("test_layers_conv", "body_conv_pool_other_dims", 4, timeout=300)


def body_transposed_general_interpolate(rank, world):
    """Transposed feature convolutions (1-3 D, kernels that do not cross worker boundaries), the
    2-D and 3-D general convolutions through the selector, channel convolutions in 1-D / 3-D form
    and the sub-tensor Interpolate module against serial torch."""
    import distdl_b200.nn as dnn
    torch.manual_seed(0)
    for nd, Pshape, xshape, Cls, fn in (
            (1, [1, 1, 4], (2, 3, 8), dnn.DistributedFeatureConvTranspose1d, torch.nn.functional.conv_transpose1d),
            (2, [1, 1, 2, 2], (2, 3, 6, 4), dnn.DistributedFeatureConvTranspose2d, torch.nn.functional.conv_transpose2d),
            (3, [1, 1, 2, 2, 1], (1, 2, 4, 4, 3), dnn.DistributedFeatureConvTranspose3d,
             torch.nn.functional.conv_transpose3d)):
        P = _cart([0, 1, 2, 3], Pshape)
        xg = _sync(torch.randn(*xshape))
        layer = Cls(P, xshape[1], 4, 2, stride=2)
        w = _sync(layer.weight.detach().clone() if rank == 0 else torch.empty(xshape[1], 4, *([2] * nd)))
        b = _sync(layer.bias.detach().clone() if rank == 0 else torch.empty(4))
        _, x = _scatter(P, xg, rank, nd + 2)
        y = _gather(P, layer(x), nd + 2)
        if rank == 0:
            assert torch.allclose(y, fn(xg, w, b, stride=2), atol=1e-5), nd
    # ---- general convolution, 2-D (space split over two workers of the pair {0, 1}) via the selector
    P_x, P_y, P_w = _cart([0, 1], [1, 1, 2, 1]), _cart([0, 1], [1, 1, 2, 1]), _cart([0, 1], [1, 1, 2, 1])
    gen = dnn.DistributedConv2d(P_x, P_y, P_w, in_channels=3, out_channels=5, kernel_size=3, padding=1)
    assert isinstance(gen, dnn.DistributedGeneralConv2d)
    x2 = _sync(torch.randn(2, 3, 12, 5))
    if rank in (0, 1):
        Wg = _sync_pair(gen.weight.detach().clone() if rank == 0 else torch.empty(5, 3, 3, 3), rank)
        bg = _sync_pair(gen.bias.detach().clone() if rank == 0 else torch.empty(5), rank)
        xl = x2[:, :, rank * 6:(rank + 1) * 6].clone()
        y = gen(xl)
        want = torch.nn.functional.conv2d(x2, Wg, bg, padding=1)[:, :, rank * 6:(rank + 1) * 6]
        assert torch.allclose(y, want, atol=1e-5)
    # ---- Interpolate on a sub-tensor: each worker produces its slab of the global result
    xg = _sync(torch.randn(1, 2, 16))
    lo, hi = rank * 4, (rank + 1) * 4
    for mode, ac in (("nearest", False), ("linear", False), ("linear", True)):
        full = torch.nn.functional.interpolate(xg, size=32, mode=mode, **({} if mode == "nearest" else
                                                                          {"align_corners": ac}))
        ylo, yhi = rank * 8, (rank + 1) * 8
        # the slab of the input that this output slab needs (one extra point on either side)
        xlo, xhi = max(0, lo - 1), min(16, hi + 1)
        mod = dnn.Interpolate([0, 0, xlo], [1, 2, xhi], [1, 2, 16], [0, 0, ylo], [1, 2, yhi], [1, 2, 32],
                              mode=mode, align_corners=ac)
        y = mod(xg[:, :, xlo:xhi].contiguous())
        assert torch.allclose(y, full[:, :, ylo:yhi], atol=1e-5), (mode, ac)
    return True


def test_transposed_general_and_interpolate():
    run_ranks("test_layers_conv", "body_transposed_general_interpolate", 4, timeout=300)


def body_collect_state_bn_conv(rank, world):
    """collect_state=True on DistributedBatchNorm (features split over 2 workers, the rest over 2)
    and DistributedFeatureConv2d: the first worker loads a serial module's tensors, the layers
    reproduce the serial module, and state_dict() returns whole tensors on the first worker only."""
    from distdl_b200.nn import DistributedBatchNorm, DistributedFeatureConv2d
    torch.manual_seed(0)
    first = rank == 0
    # batch norm, evaluation mode: uses the loaded running statistics and affine parameters
    P = _cart([0, 1, 2, 3], [2, 2, 1])
    ref = torch.nn.BatchNorm1d(6)
    with torch.no_grad():
        for t in (ref.weight, ref.bias, ref.running_mean):
            t.copy_(_sync(torch.randn(6)))
        ref.running_var.copy_(_sync(torch.rand(6) + 0.5))
    bn = DistributedBatchNorm(P, 6, collect_state=True)
    serial = {"gamma": ref.weight.detach().reshape(1, 6, 1), "beta": ref.bias.detach().reshape(1, 6, 1),
              "running_mean": ref.running_mean.reshape(1, 6, 1), "running_var": ref.running_var.reshape(1, 6, 1)}
    bn.load_state_dict({k: v.clone() for k, v in serial.items()} if first else {})
    bn.eval()
    ref.eval()
    xg = _sync(torch.randn(4, 6, 5))
    _, x = _scatter(P, xg, rank, 3)
    y = _gather(P, bn(x), 3)
    if first:
        assert torch.allclose(y, ref(xg), atol=1e-5), (y - ref(xg)).abs().max()
    sd = bn.state_dict()
    if first:
        assert list(sd) == list(serial)
        for k, v in serial.items():
            assert torch.equal(sd[k], v), k
    else:
        assert len(sd) == 0, list(sd)
    # feature convolution: the kernel lives on the first worker only
    P4 = _cart([0, 1, 2, 3], [1, 1, 2, 2])
    conv = DistributedFeatureConv2d(P4, 3, 4, 3, padding=1, collect_state=True)
    cref = torch.nn.Conv2d(3, 4, 3, padding=1)
    with torch.no_grad():
        cref.weight.copy_(_sync(cref.weight.detach().clone()))
        cref.bias.copy_(_sync(cref.bias.detach().clone()))
    conv.load_state_dict(cref.state_dict() if first else {})
    xg = _sync(torch.randn(2, 3, 8, 6))
    _, x = _scatter(P4, xg, rank, 4)
    y = _gather(P4, conv(x), 4)
    sd = conv.state_dict()
    if first:
        assert torch.allclose(y, cref(xg), atol=1e-5)
        assert torch.equal(sd["weight"], cref.weight) and torch.equal(sd["bias"], cref.bias)
    else:
        assert len(sd) == 0, list(sd)
    return True


def test_collect_state_batchnorm_and_feature_conv():
    run_ranks("test_layers_conv", "body_collect_state_bn_conv", 4, timeout=300)


def body_collect_state_channel_convs(rank, world):
    """collect_state=True on the channel all-gather / reduce-scatter convolutions, plain (1-D) and
    transposed (2-D), on [D=2, M=2, 1, ...]: a serial PyTorch module's state dict is loaded on the
    first worker, the layer reproduces the module, and state_dict() gives the tensors back there."""
    from distdl_b200 import nn
    torch.manual_seed(0)
    first = rank == 0
    d, m = rank // 2, rank % 2
    cases = [(nn.DistributedChannelAllGatherConv1d, torch.nn.Conv1d, 1, dict(padding=1)),
             (nn.DistributedChannelReduceScatterConv1d, torch.nn.Conv1d, 1, dict(padding=1)),
             (nn.DistributedChannelAllGatherConvTranspose2d, torch.nn.ConvTranspose2d, 2, dict(stride=2)),
             (nn.DistributedChannelReduceScatterConvTranspose2d, torch.nn.ConvTranspose2d, 2, dict(stride=2))]
    for cls, serial_cls, nd, kw in cases:
        P = _cart([0, 1, 2, 3], [2, 2] + [1] * nd)
        serial = serial_cls(6, 8, 3, **kw)
        with torch.no_grad():
            for t in serial.parameters():
                t.copy_(_sync(t.detach().clone()))
        layer = cls(P, 6, 8, 3, collect_state=True, **kw)
        layer.load_state_dict(serial.state_dict() if first else {})
        xg = _sync(torch.randn(4, 6, *([7] * nd)))
        y = layer(xg[d * 2:(d + 1) * 2, m * 3:(m + 1) * 3].clone())
        want = serial(xg)[d * 2:(d + 1) * 2, m * 4:(m + 1) * 4]
        assert torch.allclose(y, want, atol=1e-5), (cls.__name__, (y - want).abs().max())
        sd = layer.state_dict()
        if first:
            assert torch.equal(sd["weight"], serial.weight) and torch.equal(sd["bias"], serial.bias), cls.__name__
        else:
            assert len(sd) == 0, (cls.__name__, list(sd))
    return True


def test_collect_state_channel_convs():
    run_ranks("test_layers_conv", "body_collect_state_channel_convs", 4, timeout=300)


def body_transposed_feature_conv_general(rank, world):
    """Spatially partitioned transposed convolutions whose kernels cross worker boundaries (kernel
    larger than the stride), with padding, output padding, dilation and groups: output, input
    gradient and kernel gradient against serial PyTorch."""
    import distdl_b200.nn as dnn
    torch.manual_seed(0)
    fns = {1: torch.nn.functional.conv_transpose1d, 2: torch.nn.functional.conv_transpose2d,
           3: torch.nn.functional.conv_transpose3d}
    classes = {1: dnn.DistributedFeatureConvTranspose1d, 2: dnn.DistributedFeatureConvTranspose2d,
               3: dnn.DistributedFeatureConvTranspose3d}
    cases = [(1, [1, 1, 4], (2, 4, 11), dict(kernel_size=4, stride=2, padding=1)),
             (1, [1, 1, 4], (2, 4, 9), dict(kernel_size=3, stride=1, padding=1)),
             (1, [1, 1, 4], (1, 4, 13), dict(kernel_size=5, stride=2, padding=2, output_padding=1, groups=2)),
             (1, [1, 1, 4], (1, 4, 12), dict(kernel_size=3, stride=2, dilation=2)),
             (1, [1, 1, 4], (1, 4, 8), dict(kernel_size=2, stride=3, output_padding=2)),
             (2, [1, 1, 2, 2], (2, 4, 6, 5), dict(kernel_size=3, stride=2, padding=1, output_padding=1)),
             (2, [1, 1, 4, 1], (1, 4, 9, 4), dict(kernel_size=(4, 3), stride=(2, 1), padding=(1, 0))),
             (3, [1, 1, 2, 1, 2], (1, 4, 4, 3, 5), dict(kernel_size=3, stride=1, padding=1))]
    for nd, Pshape, xshape, kw in cases:
        P = _cart([0, 1, 2, 3], Pshape)
        layer = classes[nd](P, xshape[1], 6, **kw)
        serial = {1: torch.nn.ConvTranspose1d, 2: torch.nn.ConvTranspose2d, 3: torch.nn.ConvTranspose3d}[nd](
            xshape[1], 6, **kw)
        w = _sync(layer.weight.detach().clone() if rank == 0 else torch.empty_like(serial.weight))
        b = _sync(layer.bias.detach().clone() if rank == 0 else torch.empty(6))
        xg = _sync(torch.randn(*xshape))
        x0, x = _scatter(P, xg, rank, nd + 2)
        y = _gather(P, layer(x), nd + 2)
        fkw = {k: v for k, v in kw.items() if k != "kernel_size"}
        if rank == 0:
            xs, ws = xg.clone().requires_grad_(), w.clone().requires_grad_()
            ys = fns[nd](xs, ws, b, **fkw)
            assert y.shape == ys.shape, (kw, y.shape, ys.shape)
            assert torch.allclose(y, ys, atol=1e-5), (kw, (y - ys).abs().max())
            g = torch.randn_like(ys)
            ys.backward(g)
            y.backward(g)
            assert torch.allclose(x0.grad, xs.grad, atol=1e-5), kw
            assert torch.allclose(layer.weight.grad, ws.grad, atol=1e-4), kw
        else:
            y.backward(torch.zeros_like(y))
    return True


def test_transposed_feature_conv_crossing_worker_boundaries():
    run_ranks("test_layers_conv", "body_transposed_feature_conv_general", 4, timeout=300)


def body_conv3d_channel_and_general(rank, world):
    """3-D channel convolution (kernel blocks on a 2 x 2 grid) and 3-D general convolution (channels
    AND space split, 4 workers) through the selector, against serial conv3d: output and input gradient."""
    import torch.distributed as dist

    import distdl_b200.nn as dnn
    torch.manual_seed(0)
    # channel: P_x [1, 2, 1, 1, 1] (in), P_y [1, 2, 1, 1, 1] (out), P_w [2, 2, 1, 1, 1]
    P_x, P_y = _cart([0, 1], [1, 2, 1, 1, 1]), _cart([0, 1], [1, 2, 1, 1, 1])
    P_w = _cart([0, 1, 2, 3], [2, 2, 1, 1, 1])
    layer = dnn.DistributedConv3d(P_x, P_y, P_w, in_channels=4, out_channels=6, kernel_size=3, padding=1)
    assert isinstance(layer, dnn.DistributedChannelConv3d)
    W, b = torch.zeros(6, 4, 3, 3, 3), torch.zeros(6)
    co, ci = rank // 2, rank % 2
    W[co * 3:(co + 1) * 3, ci * 2:(ci + 1) * 2] = layer.conv_layer.weight.detach()
    if ci == 0:
        b[co * 3:(co + 1) * 3] = layer.conv_layer.bias.detach()
    dist.all_reduce(W)
    dist.all_reduce(b)
    xg = _sync(torch.randn(2, 4, 4, 5, 3))
    x0, x = _scatter(P_x, xg, rank, 5)
    y = _gather(P_y, layer(x), 5)
    if rank == 0:
        xs = xg.clone().requires_grad_()
        ys = torch.nn.functional.conv3d(xs, W, b, padding=1)
        assert torch.allclose(y, ys, atol=1e-5)
        g = torch.randn_like(ys)
        ys.backward(g)
        y.backward(g)
        assert torch.allclose(x0.grad, xs.grad, atol=1e-5)
    else:
        y.backward(torch.zeros_like(y))
    # general: input channels over 2 workers and depth over 2 workers
    P_x = _cart([0, 1, 2, 3], [1, 2, 2, 1, 1])
    P_y = _cart([0, 1], [1, 1, 2, 1, 1])            # one block of output channels: the workers with ci = 0
    P_w = _cart([0, 1, 2, 3], [1, 2, 2, 1, 1])
    gen = dnn.DistributedConv3d(P_x, P_y, P_w, in_channels=4, out_channels=4, kernel_size=3, padding=1)
    assert isinstance(gen, dnn.DistributedGeneralConv3d)
    xg = _sync(torch.randn(1, 4, 6, 4, 3))
    x0, x = _scatter(P_x, xg, rank, 5)
    # kernel blocks [co, ci / 2, 3, 3, 3] live on the workers with depth index 0 (ranks 0 and 2), the bias on rank 0
    Wg, bg = torch.zeros(4, 4, 3, 3, 3), torch.zeros(4)
    if rank in (0, 2):
        Wg[:, rank:rank + 2] = gen.weight.detach()
    if rank == 0:
        bg += gen.bias.detach()
    dist.all_reduce(Wg)
    dist.all_reduce(bg)
    yl = gen(x)
    if P_y.active:
        assert tuple(yl.shape) == (1, 4, 3, 4, 3)
    y = _gather(P_y, yl, 5)
    if rank == 0:
        xs = xg.clone().requires_grad_()
        ys = torch.nn.functional.conv3d(xs, Wg, bg, padding=1)
        assert torch.allclose(y, ys, atol=1e-5), (y - ys).abs().max()
        g = torch.randn_like(ys)
        ys.backward(g)
        y.backward(g)
        assert torch.allclose(x0.grad, xs.grad, atol=1e-5)
    else:
        y.backward(torch.zeros_like(y))
    return True


def test_conv3d_channel_and_general_via_selector():
    run_ranks("test_layers_conv", "body_conv3d_channel_and_general", 4, timeout=300)
