"""Mixture-of-experts routing ops against a dense evaluation, and the
expert-parallel block on CPU ranks."""
import math

import torch

from dist_harness import run_ranks


def test_dispatch_combine_match_dense_evaluation():
    from distdl_b200.ops import moe
    torch.manual_seed(0)
    T, d, E, k = 37, 16, 4, 2
    x = torch.randn(T, d, requires_grad=True)
    W = torch.randn(E, d, d) * 0.3
    logits = torch.randn(T, E, requires_grad=True)
    probs = torch.softmax(logits, -1)
    topw, topi = probs.topk(k, -1)
    topw = topw / topw.sum(-1, keepdim=True)
    ids = topi.to(torch.int32).reshape(-1)
    C = T * k                                     # nothing is dropped
    slot, counts = moe.assign_slots(ids, E, C)
    assert int(counts.sum()) == T * k and int((slot < 0).sum()) == 0
    buf = moe.dispatch(x, ids, slot, E, C, k)
    out = torch.einsum("ecd,efd->ecf", buf, W)
    y = moe.combine(out, topw, ids, slot, T, k)
    dense = torch.zeros(T, d)
    for c in range(k):
        dense = dense + topw[:, c:c + 1] * torch.einsum("td,tfd->tf", x, W[topi[:, c]])
    assert torch.allclose(y, dense, atol=1e-5)
    g = torch.randn_like(y)
    gx, gl = torch.autograd.grad(y, (x, logits), g, retain_graph=True)
    gx_ref, gl_ref = torch.autograd.grad(dense, (x, logits), g)
    assert torch.allclose(gx, gx_ref, atol=1e-5) and torch.allclose(gl, gl_ref, atol=1e-5)
    # a capacity limit drops the overflow pairs and nothing else
    slot2, _ = moe.assign_slots(ids, E, 5)
    for e in range(E):
        kept = ((ids == e) & (slot2 >= 0)).sum().item()
        assert kept == min(5, int(counts[e]))


def body_expert_parallel(rank, world):
    import distdl_b200  # noqa: F401
    from distdl_b200 import models
    torch.manual_seed(0)
    cfg = models.mixtral_tiny(dtype=torch.float32, n_experts=4, d_model=64, ffn_dim=96, n_heads=2, n_kv_heads=1,
                              vocab_size=200, max_seq=32, checkpoint_blocks=False)
    lay = models.ParallelLayout(world, 1)
    m = models.Decoder(cfg, lay)
    g = torch.Generator().manual_seed(10 + rank)
    tok = torch.randint(0, 200, (2, 33), generator=g)
    loss = m.loss(tok[:, :-1], tok[:, 1:])
    loss.backward()
    m.release_gathered()          # parameters kept gathered for the step deliver their gradients now
    assert math.isfinite(loss.item())
    for n, p in m.named_parameters():
        if p.numel():
            assert p.grad is not None and torch.isfinite(p.grad).all(), n
    moe = m.blocks[0].mlp
    assert moe.w_up.shape[0] == 4 // world and moe.w_up.grad.abs().sum() > 0
    return loss.item()


def test_expert_parallel_block_on_two_ranks():
    out = run_ranks("test_moe", "body_expert_parallel", 2, timeout=240)
    assert all(math.isfinite(v) for v in out)


def body_expert_layers_vs_serial(rank, world, E, N, M):
    """DistributedExpertAllGather -> GELU -> DistributedExpertReduceScatter on the grid
    [E, N, 1, M] (expert parallel x ZeRO / capacity parallel x tensor parallel) against the same
    per-expert MLP computed serially from the gathered weight shards: output and input gradient."""
    import torch.distributed as dist

    import distdl_b200
    from distdl_b200.nn import DistributedExpertAllGather, DistributedExpertReduceScatter
    experts, cap, seq, d, f = 4, 4, 2, 8, 12
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([E, N, 1, M])
    torch.manual_seed(0)
    up = DistributedExpertAllGather(P, experts, d, f, bias=True)
    down = DistributedExpertReduceScatter(P, experts, f, d, bias=True)
    ei, ni, mi = int(P.index[0]), int(P.index[1]), int(P.index[3])
    el, cl = experts // E, cap // N
    se, sc = slice(ei * el, (ei + 1) * el), slice(ni * cl, (ni + 1) * cl)
    sd = slice(mi * (d // M), (mi + 1) * (d // M))
    torch.manual_seed(1)
    X = torch.randn(experts, cap, seq, d)
    dY = torch.randn(experts, cap, seq, d)
    x = X[se, sc, :, sd].clone().requires_grad_()
    y = down(torch.nn.functional.gelu(up(x)))
    assert y.shape == (el, cl, seq, d // M)
    y.backward(dY[se, sc, :, sd])

    def gather(t):
        parts = [None] * world
        dist.all_gather_object(parts, (ei, ni, mi, None if t is None or t.numel() == 0 else t.detach().clone()))
        return parts

    # shards: W_up [e/E, in/N, out/M], W_down [e/E, out/N, in/M]; biases live on one row / column only
    Wup, Bup = torch.zeros(experts, d, f), torch.zeros(experts, 1, f)
    Wdn, Bdn = torch.zeros(experts, d, f), torch.zeros(experts, 1, d)
    for a, b, c, w in gather(up.weight):
        Wup[a * el:(a + 1) * el, b * (d // N):(b + 1) * (d // N), c * (f // M):(c + 1) * (f // M)] = w
    for a, b, c, w in gather(down.weight):
        Wdn[a * el:(a + 1) * el, b * (d // N):(b + 1) * (d // N), c * (f // M):(c + 1) * (f // M)] = w
    for a, b, c, bb in gather(up.bias):
        if bb is not None:
            Bup[a * el:(a + 1) * el, :, c * (f // M):(c + 1) * (f // M)] = bb
    for a, b, c, bb in gather(down.bias):
        if bb is not None:
            Bdn[a * el:(a + 1) * el] = bb
    Xr = X.clone().requires_grad_()
    h = torch.nn.functional.gelu(torch.einsum("ecsd,edf->ecsf", Xr, Wup) + Bup.unsqueeze(1))
    ref = torch.einsum("ecsf,edf->ecsd", h, Wdn) + Bdn.unsqueeze(1)
    ref.backward(dY)
    assert torch.allclose(y, ref[se, sc, :, sd], atol=1e-5), (y - ref[se, sc, :, sd]).abs().max()
    assert torch.allclose(x.grad, Xr.grad[se, sc, :, sd], atol=1e-5), (x.grad - Xr.grad[se, sc, :, sd]).abs().max()
    return True


def test_expert_layers_match_serial_mlp():
    run_ranks("test_moe", "body_expert_layers_vs_serial", 4, args=(2, 1, 2), timeout=180)
    run_ranks("test_moe", "body_expert_layers_vs_serial", 4, args=(1, 2, 2), timeout=180)
    run_ranks("test_moe", "body_expert_layers_vs_serial", 4, args=(2, 2, 1), timeout=180)


def body_expert_collect_state(rank, world, E, N, M, geglu):
    """collect_state=True: the first worker loads whole-layer tensors ([experts, in, out] /
    [experts, out, in], biases [experts, 1, out]); the layers then reproduce the serial per-expert
    MLP (with geglu: value * gelu(gate) on the serial halves), and state_dict() returns the same
    tensors on the first worker and nothing on the others."""
    import distdl_b200
    from distdl_b200.nn import DistributedExpertAllGather, DistributedExpertReduceScatter
    experts, cap, seq, d, f = 4, 4, 2, 8, 16
    fo = f // 2 if geglu else f
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([E, N, 1, M])
    up = DistributedExpertAllGather(P, experts, d, f, bias=True, collect_state=True, geglu=geglu)
    down = DistributedExpertReduceScatter(P, experts, fo, d, bias=True, collect_state=True)
    torch.manual_seed(3)
    Wup, Bup = torch.randn(experts, d, f), torch.randn(experts, 1, f)
    Wdn, Bdn = torch.randn(experts, d, fo), torch.randn(experts, 1, d)
    first = rank == 0
    up.load_state_dict({"weight": Wup.clone(), "bias": Bup.clone()} if first else {})
    down.load_state_dict({"weight": Wdn.clone(), "bias": Bdn.clone()} if first else {})
    ei, ni, mi = int(P.index[0]), int(P.index[1]), int(P.index[3])
    el, cl = experts // E, cap // N
    se, sc = slice(ei * el, (ei + 1) * el), slice(ni * cl, (ni + 1) * cl)
    sd = slice(mi * (d // M), (mi + 1) * (d // M))
    X = torch.randn(experts, cap, seq, d)
    h = up(X[se, sc, :, sd].clone())
    if geglu:                                   # local layout [value | gate] of this worker's share
        a, g = h.chunk(2, dim=-1)
        h = a * torch.nn.functional.gelu(g)
    else:
        h = torch.nn.functional.gelu(h)
    y = down(h)
    hr = torch.einsum("ecsd,edf->ecsf", X, Wup) + Bup.unsqueeze(1)
    if geglu:
        a, g = hr.chunk(2, dim=-1)
        hr = a * torch.nn.functional.gelu(g)
    else:
        hr = torch.nn.functional.gelu(hr)
    ref = torch.einsum("ecsf,edf->ecsd", hr, Wdn) + Bdn.unsqueeze(1)
    assert torch.allclose(y, ref[se, sc, :, sd], atol=1e-4), (y - ref[se, sc, :, sd]).abs().max()
    su, sdn = up.state_dict(), down.state_dict()
    if first:
        assert torch.equal(su["weight"], Wup) and torch.equal(su["bias"], Bup)
        assert torch.equal(sdn["weight"], Wdn) and torch.equal(sdn["bias"], Bdn)
    else:
        assert len(su) == 0 and len(sdn) == 0
    return True


def test_expert_layers_collect_state_round_trip():
    run_ranks("test_moe", "body_expert_collect_state", 4, args=(2, 1, 2, False), timeout=180)
    run_ranks("test_moe", "body_expert_collect_state", 4, args=(1, 2, 2, True), timeout=180)
    run_ranks("test_moe", "body_expert_collect_state", 4, args=(2, 2, 1, True), timeout=180)
