"""Linear-family, norm and embedding layers against serial PyTorch on CPU ranks:
weights are loaded from a serial module through the ``collect_state`` hooks,
inputs are scattered with Repartition, outputs and input gradients gathered
back and compared (the reference's vs-serial strategy,
``tests/layers/test_layernorm.py:143-265``)."""
import pytest
import torch

from dist_harness import run_ranks


def _world():
    import distdl_b200 as d
    return d.backends.backend.Partition()


def _cart(ranks, shape):
    P = _world().create_partition_inclusive(ranks)
    return P.create_cartesian_topology_partition(shape)


def _scatter_gather(P_data, gshape_dim):
    from distdl_b200.nn import Repartition
    P_root = _cart([0], [1] * gshape_dim)
    return Repartition(P_root, P_data, preserve_batch=False), Repartition(P_data, P_root, preserve_batch=False), P_root


def _run_vs_serial(layer, serial, P_in, P_out, x_global, rank, atol=1e-5, load=True):
    from distdl_b200.utilities.torch import zero_volume_tensor
    dim = x_global.dim()
    scatter, _, P_root = _scatter_gather(P_in, dim)
    _, gather, _ = _scatter_gather(P_out, dim)
    gather_dx = _scatter_gather(P_in, dim)[1]
    if load:
        sd = serial.state_dict() if P_root.active else {k: zero_volume_tensor() for k in serial.state_dict()}
        layer.load_state_dict(sd, strict=False)
    x0 = x_global.clone().requires_grad_() if P_root.active else zero_volume_tensor().requires_grad_()
    x = scatter(x0)
    y = layer(x)
    yg = gather(y)
    if P_root.active:
        xs = x_global.clone().requires_grad_()
        ys = serial(xs)
        assert yg.shape == ys.shape, (yg.shape, ys.shape)
        assert torch.allclose(yg, ys, atol=atol, rtol=1e-4), (yg - ys).abs().max()
        dy = torch.randn_like(ys)
        ys.backward(dy)
        yg.backward(dy)
        assert torch.allclose(x0.grad, xs.grad, atol=atol, rtol=1e-4), (x0.grad - xs.grad).abs().max()
    else:
        yg.backward(zero_volume_tensor())
    # round trip of the state dict in the serial layout
    out_sd = layer.state_dict()
    if P_root.active and load:
        for k, v in serial.state_dict().items():
            assert torch.allclose(out_sd[k], v), k
    return True


def body_linear_family(rank, world):
    torch.manual_seed(0)
    from distdl_b200.nn import (DistributedLinearAllGather, DistributedLinearAllGatherZero,
                                DistributedLinearReduceScatter, DistributedLinearReduceScatterZero)
    B, S, Fi, Fo = 4, 6, 16, 24
    xg = torch.randn(B, S, Fi)
    serial = torch.nn.Linear(Fi, Fo)
    P_feat = _cart([0, 1, 2, 3], [2, 1, 2])     # D=2 x M=2, features sharded
    P_seq = _cart([0, 1, 2, 3], [2, 2, 1])      # sequence sharded (sequence parallel)
    # column parallel, feature-sharded input and sequence-parallel input
    for P_x in (P_feat, P_seq):
        kw = {} if P_x is P_feat else {"P_x": P_x}
        layer = DistributedLinearAllGather(P_feat, Fi, Fo, collect_state=True, **kw)
        _run_vs_serial(layer, serial, P_x, P_feat, xg, rank)
        layer = DistributedLinearAllGatherZero(P_feat, Fi, Fo, collect_state=True, **kw)
        _run_vs_serial(layer, serial, P_x, P_feat, xg, rank)
        layer = DistributedLinearAllGatherZero(P_feat, Fi, Fo, collect_state=True, checkpoint=True, **kw)
        _run_vs_serial(layer, serial, P_x, P_feat, xg, rank)
    # row parallel, feature- and sequence-sharded output
    for P_y in (P_feat, P_seq):
        kw = {} if P_y is P_feat else {"P_y": P_y}
        layer = DistributedLinearReduceScatter(P_feat, Fi, Fo, collect_state=True, **kw)
        _run_vs_serial(layer, serial, P_feat, P_y, xg, rank)
        layer = DistributedLinearReduceScatterZero(P_feat, Fi, Fo, collect_state=True, **kw)
        _run_vs_serial(layer, serial, P_feat, P_y, xg, rank)
        layer = DistributedLinearReduceScatterZero(P_feat, Fi, Fo, collect_state=True, checkpoint=True, **kw)
        _run_vs_serial(layer, serial, P_feat, P_y, xg, rank)
    # fused QKV with grouped-query heads: serial [q | k | v] <-> per-worker [q_p | k_p | v_p]
    heads, kv, hd = 4, 2, 2
    serial = torch.nn.Linear(Fi, (heads + 2 * kv) * hd)
    layer = DistributedLinearAllGatherZero(P_feat, Fi, (heads + 2 * kv) * hd, collect_state=True, num_heads=heads,
                                           num_heads_kv=kv)
    sd = serial.state_dict()
    from distdl_b200.utilities.torch import zero_volume_tensor
    layer.load_state_dict(sd if rank == 0 else {k: zero_volume_tensor() for k in sd}, strict=False)
    out = layer.state_dict()
    if rank == 0:
        assert torch.allclose(out["weight"], sd["weight"]) and torch.allclose(out["bias"], sd["bias"])
    # the local shard holds [q_p | k_p | v_p]: check worker (d=0, m=tp) against the serial rows
    tp = rank % 2
    import torch.distributed as dist
    W = sd["weight"].clone()
    dist.broadcast(W, src=0)   # ranks drew different random numbers on the way here
    rows = torch.cat([W[tp * 4:(tp + 1) * 4], W[8 + tp * 2: 8 + (tp + 1) * 2], W[12 + tp * 2: 12 + (tp + 1) * 2]])
    d = rank // 2
    local = layer.weight.detach().reshape(Fi // 2, 8)
    assert torch.allclose(local, rows.t()[d * 8:(d + 1) * 8]), rank
    return True


def test_linear_family_vs_serial():
    run_ranks("test_layers_linear", "body_linear_family", 4, timeout=300)


def body_zero1_mode(rank, world):
    """auto_clear_buffer=False: gradients accumulate on the gathered weights over
    two micro-batches and are reduce-scattered once."""
    torch.manual_seed(0)
    from distdl_b200.nn import DistributedLinearAllGatherZero
    Fi, Fo = 8, 12
    P = _cart([0, 1, 2, 3], [2, 1, 2])
    a = DistributedLinearAllGatherZero(P, Fi, Fo, auto_clear_buffer=False)
    b = DistributedLinearAllGatherZero(P, Fi, Fo)
    b.load_state_dict(a.state_dict())
    xs = [torch.randn(2, 3, Fi // 2) for _ in range(2)]
    for x in xs:
        a(x).sum().backward()
        b(x).sum().backward()
    a.clear_weight_buffer()
    assert torch.allclose(a.weight.grad, b.weight.grad, atol=1e-6)
    assert torch.allclose(a.bias.grad, b.bias.grad, atol=1e-6)
    return True


def test_zero1_accumulation():
    run_ranks("test_layers_linear", "body_zero1_mode", 4)


def body_config1_mlp(rank, world):
    """2-layer MLP of DistributedLinear 1024->4096->1024 with GELU and
    DistributedLayerNorm(1024) on a 2x2 partition, fp32, x ~ N(0,1) [64,1024],
    MSE loss; forward and backward against the serial model."""
    torch.manual_seed(0)
    from distdl_b200.nn import DistributedLayerNorm, DistributedLinear, Repartition
    from distdl_b200.utilities.torch import zero_volume_tensor
    P_w = _cart([0, 1, 2, 3], [2, 2])
    P_x = _cart([0, 1], [1, 2])
    P_root = _cart([0], [1, 1])
    l1 = DistributedLinear(P_x, P_x, P_w, 1024, 4096)
    l2 = DistributedLinear(P_x, P_x, P_w, 4096, 1024)
    ln = DistributedLayerNorm(P_x, 1024) if rank in (0, 1) else None
    scatter, gather = Repartition(P_root, P_x, preserve_batch=False), Repartition(P_x, P_root, preserve_batch=False)
    # serial model with the same weights: gather the blocks onto rank 0
    gw = Repartition(P_w, P_root, preserve_batch=False)

    def full_weight(layer):
        return gw(layer.sublinear.weight.detach())

    def full_bias(layer, n):
        P_col = _cart([0, 2], [2, 1])
        g = Repartition(P_col, P_root, preserve_batch=False)
        b = layer.sublinear.bias.detach().reshape(-1, 1) if rank in (0, 2) else zero_volume_tensor()
        return g(b)
    W1, W2, b1, b2 = full_weight(l1), full_weight(l2), full_bias(l1, 4096), full_bias(l2, 1024)
    x_global = torch.randn(64, 1024)
    target = torch.randn(64, 1024)
    x0 = x_global.clone().requires_grad_() if rank == 0 else zero_volume_tensor().requires_grad_()
    x = scatter(x0)
    h = l1(x)
    h = torch.nn.functional.gelu(h) if rank in (0, 1) else h
    h = l2(h)
    if rank in (0, 1):
        h = ln(h)
    y = gather(h)
    if rank == 0:
        loss = torch.nn.functional.mse_loss(y, target)
        loss.backward()
        xs = x_global.clone().requires_grad_()
        hs = torch.nn.functional.linear(xs, W1, b1.reshape(-1))
        hs = torch.nn.functional.linear(torch.nn.functional.gelu(hs), W2, b2.reshape(-1))
        ys = torch.nn.functional.layer_norm(hs, (1024,))
        loss_s = torch.nn.functional.mse_loss(ys, target)
        loss_s.backward()
        err_y = (y - ys).abs().max().item()
        err_dx = (x0.grad - xs.grad).abs().max().item()
        assert err_y < 1e-4 and err_dx < 1e-5, (err_y, err_dx)
        return (err_y, err_dx)
    y.backward(torch.zeros_like(y))
    return None


def test_config1_mlp_layernorm_2x2():
    out = run_ranks("test_layers_linear", "body_config1_mlp", 4, timeout=300)
    assert out[0] is not None


def body_norms_embeddings(rank, world):
    torch.manual_seed(0)
    from distdl_b200.nn import (DistributedEmbedding, DistributedEmbeddingZero, DistributedLayerNorm,
                                DistributedLayerNormZero, DistributedRMSNormZero)
    from distdl_b200.utilities.torch import zero_volume_tensor
    B, S, F = 4, 6, 10           # 10 features over 2 workers and over 4 (ZeRO) -> uneven shards
    xg = torch.randn(B, S, F)
    P_feat = _cart([0, 1, 2, 3], [2, 1, 2])
    P_seq = _cart([0, 1, 2, 3], [2, 2, 1])
    serial = torch.nn.LayerNorm(F)
    with torch.no_grad():
        serial.weight.uniform_(0.5, 1.5)
        serial.bias.uniform_(-0.5, 0.5)
    for P in (P_feat, P_seq):
        _run_vs_serial(DistributedLayerNorm(P, F, collect_state=True), serial, P, P, xg, rank)
    _run_vs_serial(DistributedLayerNormZero(P_seq, F, collect_state=True), serial, P_seq, P_seq, xg, rank)

    class RMS(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.rand(F) + 0.5)

        def forward(self, x):
            return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * self.weight
    _run_vs_serial(DistributedRMSNormZero(P_seq, F, collect_state=True), RMS(), P_seq, P_seq, xg, rank)
    with pytest.raises(ValueError):
        DistributedRMSNormZero(P_feat, F)
    # embeddings: ids replicated over the tensor-parallel workers, table split
    V, E = 11, 6
    import torch.distributed as dist
    table = torch.randn(V, E)
    ids = torch.randint(0, V, (B, S))
    dist.broadcast(table, src=0)   # ranks consumed different amounts of random numbers above
    dist.broadcast(ids, src=0)
    P_ids = _cart([0, 1, 2, 3], [2, 2])
    for cls in (DistributedEmbedding, DistributedEmbeddingZero):
        layer = cls(P_ids, V, E, collect_state=True)
        layer.load_state_dict({"weight": table if rank == 0 else zero_volume_tensor()})
        d, m = rank // 2, rank % 2
        local_ids = ids[d * 2:(d + 1) * 2]
        out = layer(local_ids)
        want = table[local_ids][..., m * 3:(m + 1) * 3]
        assert torch.allclose(out, want), cls.__name__
        out.sum().backward()
        sd = layer.state_dict()
        if rank == 0:
            assert torch.allclose(sd["weight"], table)
    return True


def test_norms_and_embeddings():
    run_ranks("test_layers_linear", "body_norms_embeddings", 4, timeout=300)


def body_kept_buffer_goes_stale(rank, world):
    """A kept gathered buffer is re-gathered when the shard changed under it (an optimizer
    step without ``clear_weight_buffer()``), with a warning, instead of silently using the
    old weights."""
    import warnings

    import distdl_b200
    from distdl_b200.nn import DistributedLinearAllGatherZero
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([world, 1, 1])
    torch.manual_seed(0)
    lin = DistributedLinearAllGatherZero(P, 8, 6, bias=False, auto_clear_buffer=False)
    x = torch.randn(2, 3, 8)
    y0 = lin(x)
    with torch.no_grad():
        lin.weight.mul_(2.0)                              # an in-place update, as an optimizer makes
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")                  # the one-time warning about the stale copy
        y1 = lin(x)
    assert torch.allclose(y1, 2.0 * y0, atol=1e-5)
    lin.clear_weight_buffer()
    return True


def test_kept_buffer_is_regathered_after_parameter_update():
    run_ranks("test_layers_linear", "body_kept_buffer_goes_stale", 2, timeout=120)


def body_context_parallel_attention(rank, world, causal):
    """Sequence split over all workers: head <-> sequence repartitions around the local attention
    reproduce serial attention (GQA), forward and input gradients."""
    import distdl_b200
    from distdl_b200.nn import DistributedSelfAttention
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([1, world, 1, 1])
    att = DistributedSelfAttention(P, causal=causal)
    b, s, hq, hkv, d = 2, 8 * world, 2 * world, world, 16
    torch.manual_seed(4)
    Q, K, V = torch.randn(b, s, hq, d), torch.randn(b, s, hkv, d), torch.randn(b, s, hkv, d)
    dO = torch.randn(b, s, hq, d)
    sl = slice(rank * (s // world), (rank + 1) * (s // world))
    q, k, v = (t[:, sl].clone().requires_grad_() for t in (Q, K, V))
    out = att(q, k, v)
    out.backward(dO[:, sl])
    Qr, Kr, Vr = (t.clone().requires_grad_() for t in (Q, K, V))
    rep = hq // hkv
    ref = torch.nn.functional.scaled_dot_product_attention(
        Qr.transpose(1, 2), Kr.transpose(1, 2).repeat_interleave(rep, 1), Vr.transpose(1, 2).repeat_interleave(rep, 1),
        is_causal=causal).transpose(1, 2)
    ref.backward(dO)
    assert torch.allclose(out, ref[:, sl], atol=1e-5), (out - ref[:, sl]).abs().max()
    for got, want in ((q.grad, Qr.grad), (k.grad, Kr.grad), (v.grad, Vr.grad)):
        assert torch.allclose(got, want[:, sl], atol=1e-5), (got - want[:, sl]).abs().max()
    return True


def test_context_parallel_attention_matches_serial():
    run_ranks("test_layers_linear", "body_context_parallel_attention", 2, args=(True,), timeout=120)
    run_ranks("test_layers_linear", "body_context_parallel_attention", 4, args=(False,), timeout=120)


def body_ring_attention(rank, world, causal, hq, hkv, zigzag=False):
    """K / V blocks travel around the ring; result and all three gradients equal serial attention
    (head counts need not divide by the ring size)."""
    import distdl_b200
    from distdl_b200.nn import DistributedRingAttention
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([1, world, 1, 1])
    att = DistributedRingAttention(P, causal=causal, zigzag=zigzag)
    b, s, d = 2, 6 * world, 16
    torch.manual_seed(9)
    Q, K, V = torch.randn(b, s, hq, d), torch.randn(b, s, hkv, d), torch.randn(b, s, hkv, d)
    dO = torch.randn(b, s, hq, d)
    sl = slice(rank * (s // world), (rank + 1) * (s // world))
    if zigzag:                                  # chunks rank and 2 * world - 1 - rank of the 2 * world chunks
        c = s // (2 * world)
        hi = 2 * world - 1 - rank
        sl = list(range(rank * c, (rank + 1) * c)) + list(range(hi * c, (hi + 1) * c))
    q, k, v = (t[:, sl].clone().requires_grad_() for t in (Q, K, V))
    out = att(q, k, v)
    out.backward(dO[:, sl])
    Qr, Kr, Vr = (t.clone().requires_grad_() for t in (Q, K, V))
    rep = hq // hkv
    ref = torch.nn.functional.scaled_dot_product_attention(
        Qr.transpose(1, 2), Kr.transpose(1, 2).repeat_interleave(rep, 1), Vr.transpose(1, 2).repeat_interleave(rep, 1),
        is_causal=causal).transpose(1, 2)
    ref.backward(dO)
    assert torch.allclose(out, ref[:, sl], atol=2e-5), (out - ref[:, sl]).abs().max()
    for got, want, what in ((q.grad, Qr.grad, "dq"), (k.grad, Kr.grad, "dk"), (v.grad, Vr.grad, "dv")):
        assert torch.allclose(got, want[:, sl], atol=2e-5), (what, (got - want[:, sl]).abs().max())
    return True


def test_ring_attention_matches_serial():
    run_ranks("test_layers_linear", "body_ring_attention", 3, args=(True, 4, 2), timeout=180)
    run_ranks("test_layers_linear", "body_ring_attention", 4, args=(False, 3, 3), timeout=180)
    # the load-balanced layout: two chunks per worker, same result
    run_ranks("test_layers_linear", "body_ring_attention", 3, args=(True, 4, 2, True), timeout=180)
    run_ranks("test_layers_linear", "body_ring_attention", 4, args=(True, 3, 3, True), timeout=180)
    run_ranks("test_layers_linear", "body_ring_attention", 2, args=(False, 2, 2, True), timeout=180)


def body_init(rank, world):
    """Xavier / Kaiming initialisers take their fans from the GLOBAL tensor: a [64, 32] weight
    split over 4 workers gets the bound of the unsplit weight, on every worker."""
    import math

    import distdl_b200
    from distdl_b200.nn import init
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([2, 2])
    torch.manual_seed(rank)
    w = torch.empty(32, 16)                                 # local shard of the [64, 32] weight
    init.xavier_uniform_(P, w)
    bound = math.sqrt(3.0) * math.sqrt(2.0 / (32 + 64))
    assert w.abs().max() <= bound + 1e-6 and w.abs().max() > 0.8 * bound
    init.kaiming_uniform_(P, w, a=math.sqrt(5))
    kb = math.sqrt(3.0) * math.sqrt(2.0 / (1 + 5)) / math.sqrt(32)      # fan_in of the global weight = 32
    assert w.abs().max() <= kb + 1e-6 and w.abs().max() > 0.8 * kb
    init.xavier_normal_(P, w)
    assert abs(w.std().item() - math.sqrt(2.0 / 96)) < 0.02
    init.kaiming_normal_(P, w, mode="fan_out", nonlinearity="relu")
    assert abs(w.std().item() - math.sqrt(2.0 / 64)) < 0.03
    z = torch.empty(0)
    assert init.xavier_uniform_(P, torch.empty(32, 16)[:0]).numel() == 0 and z.numel() == 0
    init.zeros_(w)
    assert float(w.abs().sum()) == 0.0
    return True


def test_initialisers_use_global_fans():
    run_ranks("test_layers_linear", "body_init", 4, timeout=120)


def body_window_attention(rank, world, window, hq, hkv):
    """Sliding-window causal attention with the previous block's last keys fetched by halo exchange:
    output and all three gradients equal serial banded attention."""
    import distdl_b200
    from distdl_b200.nn import DistributedSlidingWindowAttention
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([1, world, 1, 1])
    att = DistributedSlidingWindowAttention(P, window)
    b, s, d = 2, 6 * world, 8
    torch.manual_seed(4)
    Q, K, V = torch.randn(b, s, hq, d), torch.randn(b, s, hkv, d), torch.randn(b, s, hkv, d)
    dO = torch.randn(b, s, hq, d)
    sl = slice(rank * 6, (rank + 1) * 6)
    q, k, v = (t[:, sl].clone().requires_grad_() for t in (Q, K, V))
    out = att(q, k, v)
    out.backward(dO[:, sl])
    Qr, Kr, Vr = (t.clone().requires_grad_() for t in (Q, K, V))
    i, j = torch.arange(s).unsqueeze(1), torch.arange(s).unsqueeze(0)
    band = (j <= i) & (j > i - window)
    rep = hq // hkv
    ref = torch.nn.functional.scaled_dot_product_attention(
        Qr.transpose(1, 2), Kr.transpose(1, 2).repeat_interleave(rep, 1), Vr.transpose(1, 2).repeat_interleave(rep, 1),
        attn_mask=band).transpose(1, 2)
    ref.backward(dO)
    assert torch.allclose(out, ref[:, sl], atol=2e-5), (out - ref[:, sl]).abs().max()
    for got, want, what in ((q.grad, Qr.grad, "dq"), (k.grad, Kr.grad, "dk"), (v.grad, Vr.grad, "dv")):
        assert torch.allclose(got, want[:, sl], atol=2e-5), (what, (got - want[:, sl]).abs().max())
    return True


def test_sliding_window_attention_by_halo_exchange():
    run_ranks("test_layers_linear", "body_window_attention", 4, args=(4, 4, 2), timeout=180)
    run_ranks("test_layers_linear", "body_window_attention", 3, args=(7, 2, 2), timeout=180)
    run_ranks("test_layers_linear", "body_window_attention", 2, args=(1, 2, 1), timeout=180)


def body_store_bias_partition(rank, world):
    """A user-supplied ``P_store_bias`` (here the second data-parallel row instead of the first) carries
    the bias between the shards and the serial state dict."""
    from distdl_b200.nn import DistributedLinearAllGatherZero
    from distdl_b200.utilities.torch import zero_volume_tensor
    torch.manual_seed(0)
    P_feat = _cart([0, 1, 2, 3], [2, 1, 2])
    P_store = _cart([2, 3], [1, 2, 1])
    serial = torch.nn.Linear(10, 12)
    layer = DistributedLinearAllGatherZero(P_feat, 10, 12, collect_state=True, P_store_bias=P_store)
    sd = serial.state_dict() if rank == 0 else {k: zero_volume_tensor() for k in serial.state_dict()}
    layer.load_state_dict(sd, strict=False)
    out = layer.state_dict()
    if rank == 0:
        for k, v in serial.state_dict().items():
            assert torch.allclose(out[k], v), k
    xg = torch.randn(4, 3, 10)
    _run_vs_serial(layer, serial, P_feat, P_feat, xg, rank, load=False)
    # a member that sits in the wrong tensor-parallel column is refused
    bad = _cart([3, 2], [1, 2, 1])
    try:
        DistributedLinearAllGatherZero(P_feat, 10, 12, P_store_bias=bad)
        ok = rank not in (2, 3)
    except ValueError:
        ok = rank in (2, 3)
    assert ok
    return True


def test_store_bias_partition_is_honoured():
    run_ranks("test_layers_linear", "body_store_bias_partition", 4, timeout=120)
