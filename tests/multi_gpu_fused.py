"""Fused all-gather->GEMM and GEMM->reduce-scatter against the unfused NCCL +
fp32 reference, forward and backward."""
import torch
import torch.distributed as dist


def check_fused():
    from distdl_b200 import _native
    from distdl_b200.parallel import fused
    world, rank = dist.get_world_size(), dist.get_rank()
    ranks = tuple(range(world))
    dev = torch.device("cuda", torch.cuda.current_device())
    for (b, s_local, K, N) in [(1, 128, 256, 512), (2, 256, 1024, 768), (2, 1024, 4096, 3072)]:
        for trial in range(2):
            torch.manual_seed(1000 + trial)            # same weights everywhere
            w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
            bias = (torch.randn(N, device=dev) * 0.1).to(torch.bfloat16).requires_grad_()
            torch.manual_seed(rank * 7 + trial)
            x = torch.randn(b, s_local, K, device=dev).to(torch.bfloat16).requires_grad_()
            # ---- all-gather -> GEMM
            y = fused.AgLinearFn.apply(x, w, bias, ranks)
            xs = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(xs, x.detach())
            xg = torch.cat(xs, dim=1).float()
            ref = xg @ w.detach().float().t() + bias.detach().float()
            err = (y.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
            assert err < 2e-2, ("ag_gemm fwd", b, s_local, K, N, err)
            dy = torch.randn_like(y)
            y.backward(dy)
            dxg = dy.float() @ w.detach().float()                      # [b, P*s_local, K] partial of this member
            dist.all_reduce(dxg)
            dx_ref = dxg[:, rank * s_local:(rank + 1) * s_local]
            err = (x.grad.float() - dx_ref).abs().max().item() / (dx_ref.abs().max().item() + 1e-6)
            assert err < 3e-2, ("ag_gemm dx", b, s_local, K, N, err)
            dw_ref = dy.reshape(-1, N).float().t() @ xg.reshape(-1, K)
            err = (w.grad.float() - dw_ref).abs().max().item() / (dw_ref.abs().max().item() + 1e-6)
            assert err < 3e-2, ("ag_gemm dw", err)
            # ---- GEMM -> reduce-scatter (row parallel: K is this member's feature slice)
            w2 = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
            xin = torch.randn(b, world * s_local, K, device=dev).to(torch.bfloat16).requires_grad_()
            out = fused.LinearRsFn.apply(xin, w2, bias.detach() if rank == 0 else None, ranks)
            full = xin.detach().float() @ w2.detach().float().t()
            if rank == 0:
                full = full + bias.detach().float()
            dist.all_reduce(full)
            ref = full[:, rank * s_local:(rank + 1) * s_local]
            err = (out.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
            assert err < 3e-2, ("gemm_rs fwd", b, s_local, K, N, err)
            dyl = torch.randn_like(out)
            out.backward(dyl)
            dys = [torch.empty_like(dyl) for _ in range(world)]
            dist.all_gather(dys, dyl)
            dyg = torch.cat(dys, dim=1).float()
            dx_ref = dyg @ w2.detach().float()
            err = (xin.grad.float() - dx_ref).abs().max().item() / (dx_ref.abs().max().item() + 1e-6)
            assert err < 3e-2, ("gemm_rs dx", err)
            dw_ref = dyg.reshape(-1, N).t() @ xin.detach().reshape(-1, K).float()
            err = (w2.grad.float() - dw_ref).abs().max().item() / (dw_ref.abs().max().item() + 1e-6)
            assert err < 3e-2, ("gemm_rs dw", err)
    # ---- shards of different lengths that are no multiple of 128 rows (3 * 128 + 77 and one less):
    # the padded forms of both fused operators, forward and backward
    b, K, N = 2, 512, 768
    S = 461 * world - 1
    extents = fused._balanced(S, world)
    s_pad = -(-max(extents) // 128) * 128
    s_me, lo = extents[rank], sum(extents[:rank])
    torch.manual_seed(77)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
    bias = (torch.randn(N, device=dev) * 0.1).to(torch.bfloat16).requires_grad_()
    xfull = torch.randn(b, S, K, device=dev).to(torch.bfloat16)            # the same on every member
    x = xfull[:, lo:lo + s_me].clone().requires_grad_()
    y = fused.AgLinearPaddedFn.apply(x, w, bias, ranks, tuple(extents), s_pad)
    ref = xfull.float() @ w.detach().float().t() + bias.detach().float()
    assert y.shape == ref.shape
    err = (y.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
    assert err < 2e-2, ("padded ag_gemm fwd", err)
    torch.manual_seed(500 + rank)
    dy = torch.randn_like(y)
    y.backward(dy)
    dxg = dy.float() @ w.detach().float()
    dist.all_reduce(dxg)
    err = (x.grad.float() - dxg[:, lo:lo + s_me]).abs().max().item() / (dxg.abs().max().item() + 1e-6)
    assert err < 3e-2, ("padded ag_gemm dx", err)
    dw_ref = dy.reshape(-1, N).float().t() @ xfull.reshape(-1, K).float()
    err = (w.grad.float() - dw_ref).abs().max().item() / (dw_ref.abs().max().item() + 1e-6)
    assert err < 3e-2, ("padded ag_gemm dw", err)
    w2 = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16).requires_grad_()
    torch.manual_seed(900 + rank)
    xin = torch.randn(b, S, K, device=dev).to(torch.bfloat16).requires_grad_()
    out = fused.LinearRsPaddedFn.apply(xin, w2, None, ranks, tuple(extents), s_pad, rank)
    full = xin.detach().float() @ w2.detach().float().t()
    dist.all_reduce(full)
    err = (out.float() - full[:, lo:lo + s_me]).abs().max().item() / (full.abs().max().item() + 1e-6)
    assert out.shape == (b, s_me, N) and err < 3e-2, ("padded gemm_rs fwd", err)
    dyl = torch.randn_like(out)
    out.backward(dyl)
    dys = [torch.empty(b, e, N, dtype=dyl.dtype, device=dev) for e in extents]
    dist.all_gather(dys, dyl) if len(set(extents)) == 1 else [
        dist.broadcast(t if r != rank else t.copy_(dyl), src=r) for r, t in enumerate(dys)]
    dyg = torch.cat(dys, dim=1).float()
    dx_ref = dyg @ w2.detach().float()
    err = (xin.grad.float() - dx_ref).abs().max().item() / (dx_ref.abs().max().item() + 1e-6)
    assert err < 3e-2, ("padded gemm_rs dx", err)
    dw_ref = dyg.reshape(-1, N).t() @ xin.detach().reshape(-1, K).float()
    err = (w2.grad.float() - dw_ref).abs().max().item() / (dw_ref.abs().max().item() + 1e-6)
    assert err < 3e-2, ("padded gemm_rs dw", err)
    # ---- GEMM -> reduce-scatter: run-to-run determinism, and an error bound that follows the team size.
    # The partial products travel as bf16 and are folded in fp32 in member order, so every output
    # element is the fp32 sum of P values each within one bf16 rounding of its exact partial: the error
    # is bounded by sum_i |partial_i| * 2^-8 (plus the final rounding of the result), whatever P is.
    b, s_local, K, N = 2, 256, 2048, 1024
    torch.manual_seed(31)
    w3 = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    torch.manual_seed(300 + rank)
    x3 = torch.randn(b, world * s_local, K, device=dev).to(torch.bfloat16)
    first = fused.gemm_rs(x3.reshape(-1, K), w3, None, ranks, b, s_local)
    again = fused.gemm_rs(x3.reshape(-1, K), w3, None, ranks, b, s_local)
    assert torch.equal(first, again), "gemm_rs is not deterministic from run to run"
    part = x3.double() @ w3.double().t()                                   # this member's exact partial
    total, mag = part.clone(), part.abs()
    dist.all_reduce(total)
    dist.all_reduce(mag)
    sl = slice(rank * s_local, (rank + 1) * s_local)
    bound = mag[:, sl] * 2.0 ** -8 + total[:, sl].abs() * 2.0 ** -8 + 1e-3
    excess = ((first.double() - total[:, sl]).abs() - bound).max().item()
    assert excess <= 0, ("gemm_rs error beyond the bf16-partial bound", world, excess)
    # back-to-back calls without synchronisation in between: the shard staging is double
    # buffered, so a call must never overwrite a shard that a slower peer still reads
    b, s_local, K, N = 2, 512, 2048, 1024
    torch.manual_seed(5)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    torch.manual_seed(100 + rank)
    xs_local = [torch.randn(b, s_local, K, device=dev).to(torch.bfloat16) for _ in range(7)]
    outs = []
    for i, x in enumerate(xs_local):
        if i % 3 == rank % 3:
            torch.cuda._sleep(2_000_000)               # skew the members against each other
        outs.append(fused.ag_gemm(x, w, None, ranks))
    for x, (y, G) in zip(xs_local, outs):
        xs = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(xs, x)
        xg = torch.cat(xs, dim=1)
        assert torch.equal(G, xg), "gathered activation differs"
        ref = xg.float() @ w.float().t()
        err = (y.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-6)
        assert err < 2e-2, ("ag_gemm back-to-back", err)
    torch.cuda.synchronize()
    assert _native.read_status()[0] == 0, _native.read_status()
