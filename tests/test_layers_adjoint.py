"""Adjoint (dot-product) tests per layer, as the reference runs them for the input, the weight and
the bias of every layer (``tests/layers/test_linear_ag.py:351-427`` and its siblings): with the
other operands fixed, a layer is linear in its input, in its weight and in its bias, so
``<F(v), dy> == <v, F*(dy)>`` must hold with the inner products summed over ALL workers --
including workers that are not part of the layer's partition and hold zero-volume tensors."""
import torch

from adjoint_test import check_adjoint_test_tight
from dist_harness import run_ranks


def _cart(ranks, shape):
    import distdl_b200 as d
    P = d.backends.backend.Partition().create_partition_inclusive(ranks)
    return P.create_cartesian_topology_partition(shape)


def _params(layer):
    w = [p for n, p in layer.named_parameters() if "weight" in n]
    b = [p for n, p in layer.named_parameters() if "bias" in n]
    return w, b


def _adjoints(make_layer, make_input, active, has_bias=True, rtol=1e-5):
    """Input and weight adjoints on a layer without bias, bias adjoint on a layer with bias and a
    zero input.  ``make_input()`` gives this worker's input (zero-volume where it holds none)."""
    from distdl_b200.utilities.torch import zero_volume_tensor
    torch.manual_seed(0)
    layer = make_layer(False).double()
    x = make_input().double().requires_grad_()
    y = layer(x)
    dy = torch.randn_like(y)
    if y.requires_grad:
        y.backward(dy)
    if hasattr(layer, "clear_weight_buffer"):
        layer.clear_weight_buffer()
    dx = x.grad if x.grad is not None else zero_volume_tensor(dtype=torch.float64)
    check_adjoint_test_tight(x.detach(), dx, y.detach(), dy, rtol=rtol)
    ws, _ = _params(layer)
    W = torch.cat([p.detach().reshape(-1) for p in ws]) if ws else zero_volume_tensor(dtype=torch.float64)
    dW = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in ws]) if ws else W
    check_adjoint_test_tight(W, dW, y.detach(), dy, rtol=rtol)
    if not has_bias:
        return
    layer = make_layer(True).double()
    ws, bs = _params(layer)
    with torch.no_grad():
        for p in ws:
            p.zero_()
    x = torch.zeros_like(make_input().double())
    y = layer(x)
    dy = torch.randn_like(y)
    if y.requires_grad:
        y.backward(dy)
    if hasattr(layer, "clear_weight_buffer"):
        layer.clear_weight_buffer()
    B = torch.cat([p.detach().reshape(-1) for p in bs]) if bs else zero_volume_tensor(dtype=torch.float64)
    dB = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in bs]) if bs else B
    check_adjoint_test_tight(B, dB, y.detach(), dy, rtol=rtol)


def body_linear_adjoints(rank, world):
    """Six workers, four of them in the layer (workers 4 and 5 are inactive)."""
    from distdl_b200 import nn as dnn
    from distdl_b200.utilities.slicing import compute_subshape
    from distdl_b200.utilities.torch import zero_volume_tensor
    active = rank < 4
    P_feat = _cart([0, 1, 2, 3], [2, 1, 2])
    P_seq = _cart([0, 1, 2, 3], [2, 2, 1])
    B, S, Fi, Fo = 4, 6, 10, 14        # 10 and 14 do not divide evenly everywhere

    def local(P, gshape):
        if not P.active:
            return zero_volume_tensor()
        return torch.randn(*[int(v) for v in compute_subshape(P.shape, P.index, gshape)])

    for cls, kw, P_in in ((dnn.DistributedLinearAllGather, {}, P_feat),
                          (dnn.DistributedLinearAllGather, {"P_x": P_seq}, P_seq),
                          (dnn.DistributedLinearAllGatherZero, {}, P_feat),
                          (dnn.DistributedLinearAllGatherZero, {"P_x": P_seq, "checkpoint": True}, P_seq),
                          (dnn.DistributedLinearAllGatherZero, {"auto_clear_buffer": False}, P_feat),
                          (dnn.DistributedLinearReduceScatter, {}, P_feat),
                          (dnn.DistributedLinearReduceScatter, {"P_y": P_seq}, P_feat),
                          (dnn.DistributedLinearReduceScatterZero, {}, P_feat),
                          (dnn.DistributedLinearReduceScatterZero, {"P_y": P_seq, "checkpoint": True}, P_feat)):
        _adjoints(lambda bias: cls(P_feat, Fi, Fo, bias=bias, **kw), lambda: local(P_in, [B, S, Fi]), active)
    # the general 2-D layer: P_x [1, 2], P_y [1, 2], P_w [2, 2]
    P_x, P_w = _cart([0, 1], [1, 2]), _cart([0, 1, 2, 3], [2, 2])
    _adjoints(lambda bias: dnn.DistributedLinear(P_x, P_x, P_w, Fi, Fo, bias=bias), lambda: local(P_x, [B, Fi]),
              rank < 2)
    return True


def body_other_adjoints(rank, world):
    from distdl_b200 import nn as dnn
    from distdl_b200.utilities.slicing import compute_subshape
    from distdl_b200.utilities.torch import zero_volume_tensor
    active = rank < 4

    def local(P, gshape):
        if not P.active:
            return zero_volume_tensor()
        return torch.randn(*[int(v) for v in compute_subshape(P.shape, P.index, gshape)])

    # feature-space convolution over a 2 x 2 spatial grid (halo exchange inside)
    P_sp = _cart([0, 1, 2, 3], [1, 1, 2, 2])
    _adjoints(lambda bias: dnn.DistributedFeatureConv2d(P_sp, 3, 4, 3, padding=1, bias=bias),
              lambda: local(P_sp, [2, 3, 9, 10]), active)
    _adjoints(lambda bias: dnn.DistributedFeatureConv2d(P_sp, 3, 4, 3, stride=2, padding=1, bias=bias),
              lambda: local(P_sp, [2, 3, 9, 10]), active)
    # channel-parallel convolutions on [D = 2, M = 2, 1]
    P_ch = _cart([0, 1, 2, 3], [2, 2, 1])
    _adjoints(lambda bias: dnn.DistributedChannelAllGatherConv1d(P_ch, 6, 8, 3, padding=1, bias=bias),
              lambda: local(P_ch, [4, 6, 9]), active)
    _adjoints(lambda bias: dnn.DistributedChannelReduceScatterConv1d(P_ch, 6, 8, 3, padding=1, bias=bias),
              lambda: local(P_ch, [4, 6, 9]), active)
    # general convolution: channels in / out on a 2 x 2 weight grid
    P_x, P_y, P_w = _cart([0, 1], [1, 2, 1]), _cart([0, 1], [1, 2, 1]), _cart([0, 1, 2, 3], [2, 2, 1])
    _adjoints(lambda bias: dnn.DistributedConv1d(P_x, P_y, P_w, in_channels=4, out_channels=6, kernel_size=3,
                                                 padding=1, bias=bias),
              lambda: local(P_x, [2, 4, 7]), rank < 2)
    # the norm layers are linear in their weight and bias (not in their input)
    P_feat, P_seq = _cart([0, 1, 2, 3], [2, 1, 2]), _cart([0, 1, 2, 3], [2, 2, 1])
    for make, P_n in ((lambda: dnn.DistributedLayerNorm(P_feat, 12), P_feat),
                      (lambda: dnn.DistributedLayerNormZero(P_seq, 12), P_seq)):
        torch.manual_seed(1)
        layer = make().double()
        x = local(P_n, [4, 5, 12]).double()
        for name in ("weight", "bias"):
            with torch.no_grad():
                for n, p in layer.named_parameters():
                    p.copy_(torch.randn_like(p)) if n == name else p.zero_()
            layer.zero_grad()
            y = layer(x)
            dy = torch.randn_like(y)
            if y.requires_grad:
                y.backward(dy)
            if hasattr(layer, "clear_weight_buffer"):
                layer.clear_weight_buffer()
            ps = [p for n, p in layer.named_parameters() if n == name]
            V = torch.cat([p.detach().reshape(-1) for p in ps]) if ps else zero_volume_tensor(dtype=torch.float64)
            dV = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in ps]) \
                if ps else V
            check_adjoint_test_tight(V, dV, y.detach(), dy, rtol=1e-5)
    # the embedding is linear in its table
    P_e = _cart([0, 1, 2, 3], [2, 2])
    for cls in (dnn.DistributedEmbedding, dnn.DistributedEmbeddingZero):
        torch.manual_seed(2)
        layer = cls(P_e, 20, 12).double()
        if active:
            ids = torch.randint(0, 20, (3, 4), generator=torch.Generator().manual_seed(rank // 2))
        else:
            ids = zero_volume_tensor(dtype=torch.int64)
        y = layer(ids)
        dy = torch.randn_like(y)
        if y.requires_grad:
            y.backward(dy)
        if hasattr(layer, "clear_weight_buffer"):
            layer.clear_weight_buffer()
        ps = list(layer.parameters())
        V = torch.cat([p.detach().reshape(-1) for p in ps]) if ps else zero_volume_tensor(dtype=torch.float64)
        dV = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in ps]) if ps else V
        check_adjoint_test_tight(V, dV, y.detach(), dy, rtol=1e-5)
    return True


def body_expert_pool_upsample_adjoints(rank, world):
    """Expert layers (input / weight / bias), average pooling, up-sampling and the transposed feature
    convolution (all linear in their input): six workers, four in the layer."""
    from distdl_b200 import nn as dnn
    from distdl_b200.utilities.slicing import compute_subshape
    from distdl_b200.utilities.torch import zero_volume_tensor
    active = rank < 4

    def local(P, gshape):
        if not P.active:
            return zero_volume_tensor()
        return torch.randn(*[int(v) for v in compute_subshape(P.shape, P.index, gshape)])

    # expert layers on [E = 2, N = 1, 1, M = 2]: experts x capacity x sequence x features
    P_e = _cart([0, 1, 2, 3], [2, 1, 1, 2])
    experts, cap, seq, d, f = 4, 3, 2, 8, 12
    _adjoints(lambda bias: dnn.DistributedExpertAllGather(P_e, experts, d, f, bias=bias),
              lambda: local(P_e, [experts, cap, seq, d]), active)
    _adjoints(lambda bias: dnn.DistributedExpertReduceScatter(P_e, experts, f, d, bias=bias),
              lambda: local(P_e, [experts, cap, seq, f]), active)
    # layers without parameters: the input adjoint alone
    P_sp = _cart([0, 1, 2, 3], [1, 1, 2, 2])
    for make, gshape in ((lambda: dnn.DistributedAvgPool2d(P_sp, kernel_size=2, stride=2), [2, 3, 8, 12]),
                         (lambda: dnn.DistributedAvgPool2d(P_sp, kernel_size=3, stride=1, padding=1), [2, 3, 7, 9]),
                         (lambda: dnn.DistributedUpsample(P_sp, scale_factor=2, mode="linear"), [2, 3, 5, 6]),
                         (lambda: dnn.DistributedUpsample(P_sp, size=[9, 11], mode="nearest"), [2, 3, 5, 6])):
        torch.manual_seed(3)
        layer = make()
        x = local(P_sp, gshape).double().requires_grad_()
        y = layer(x)
        dy = torch.randn_like(y)
        if y.requires_grad:
            y.backward(dy)
        dx = x.grad if x.grad is not None else zero_volume_tensor(dtype=torch.float64)
        check_adjoint_test_tight(x.detach(), dx, y.detach(), dy, rtol=1e-5)
    # transposed feature convolution (halo accumulate inside)
    _adjoints(lambda bias: dnn.DistributedFeatureConvTranspose2d(P_sp, 3, 4, 3, stride=2, padding=1, bias=bias),
              lambda: local(P_sp, [2, 3, 6, 8]), active)
    return True


def test_linear_family_adjoints_with_inactive_workers():
    run_ranks("test_layers_adjoint", "body_linear_adjoints", 6, timeout=300)


def test_conv_norm_and_embedding_adjoints_with_inactive_workers():
    run_ranks("test_layers_adjoint", "body_other_adjoints", 6, timeout=300)


def test_expert_pooling_upsampling_and_transposed_conv_adjoints():
    run_ranks("test_layers_adjoint", "body_expert_pool_upsample_adjoints", 6, timeout=300)
