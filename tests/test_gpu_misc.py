"""Interpolation and MoE routing kernels on the GPU against their CPU /
PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("nd,mode,ac", [(1, "linear", False), (2, "linear", True), (3, "linear", False),
                                        (2, "nearest", False)])
def test_interpolate_cuda_matches_cpu_oracle(nd, mode, ac):
    from distdl_b200.functional.interpolate import interpolate
    torch.manual_seed(0)
    ins, outs = [9, 7, 6][:nd], [20, 15, 11][:nd]
    x = torch.randn(3, 4, *ins)
    # a slab of the output computed from a slab of the input, in global coordinates
    x_lo = [2] + [0] * (nd - 1)
    y_lo = [8] + [0] * (nd - 1)
    xs = x[:, :, 2:].contiguous()
    args = (x_lo, ins, ins, y_lo, outs, outs, None, mode, ac)
    xc = xs.clone().requires_grad_()
    yc = interpolate(xc, *args)
    xg = xs.cuda().requires_grad_()
    yg = interpolate(xg, *args)
    assert torch.allclose(yg.cpu(), yc, atol=1e-5)
    g = torch.randn_like(yc)
    yc.backward(g)
    yg.backward(g.cuda())
    assert torch.allclose(xg.grad.cpu(), xc.grad, atol=1e-4)


def test_moe_routing_kernels_match_torch():
    from distdl_b200.ops import moe
    torch.manual_seed(0)
    T, d, E, k, C = 300, 256, 8, 2, 96
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, E, (T * k,), device="cuda", dtype=torch.int32)
    w = torch.rand(T, k, device="cuda", requires_grad=True)
    slot, counts = moe.assign_slots(ids, E, C)
    assert int(counts.sum()) == T * k
    ref_slot, ref_counts = moe.assign_slots(ids.cpu(), E, C)
    assert torch.equal(slot.cpu(), ref_slot) and torch.equal(counts.cpu(), ref_counts)
    for e in range(E):
        s = slot[(ids == e)]
        kept = s[s >= 0]
        assert kept.numel() == min(C, int(counts[e])) and kept.unique().numel() == kept.numel()
    buf = moe.dispatch(x, ids, slot, E, C, k)
    y = moe.combine(buf * 2, w, ids, slot, T, k)
    keep = (slot >= 0).reshape(T, k).float()
    ref = (2 * x.detach().float()) * (w.detach() * keep).sum(1, keepdim=True)
    assert (y.float() - ref).abs().max().item() < 3e-2 * ref.abs().max().item()
    g = torch.randn_like(y)
    y.backward(g)
    gx_ref = 2 * g.float() * (w.detach() * keep).sum(1, keepdim=True)
    assert (x.grad.float() - gx_ref).abs().max().item() < 3e-2 * gx_ref.abs().max().item()
    gw_ref = (2 * x.detach().float() * g.float()).sum(1, keepdim=True) * keep
    assert (w.grad - gw_ref).abs().max().item() < 3e-2 * gw_ref.abs().max().item() + 1e-3


@pytest.mark.parametrize("E,k,ld", [(8, 2, 8), (6, 1, 8), (16, 4, 16), (40, 8, 40), (64, 2, 64)])
def test_router_kernel_matches_softmax_topk_renormalisation(E, k, ld):
    """The router kernels (softmax, top-k, renormalised weights, probability sums; slots in pair-index
    order) and the backward kernel against the same computation written with PyTorch ops in fp32."""
    from distdl_b200.ops import moe
    torch.manual_seed(E * 10 + k)
    T, C = 777, 10_000
    logits = (torch.randn(T, ld, device="cuda") * 2).to(torch.bfloat16).requires_grad_()
    w, prob_sum, ids, slot, counts = moe.route(logits, E, k, C)
    lr = logits.detach().float()[:, :E].requires_grad_()
    probs = torch.softmax(lr, dim=-1)
    topw, topi = probs.topk(k, dim=-1)
    topw = topw / topw.sum(-1, keepdim=True)
    assert torch.equal(ids.reshape(T, k).long().sort(-1).values, topi.sort(-1).values)
    order = ids.reshape(T, k).long().argsort(-1), topi.argsort(-1)
    assert torch.allclose(w.gather(1, order[0]), topw.gather(1, order[1]), atol=1e-5)
    assert torch.allclose(prob_sum, probs.sum(0), rtol=1e-4, atol=1e-3)
    assert torch.equal(counts.long(), torch.bincount(ids.long(), minlength=E))
    # every pair has its own slot within its expert (nothing dropped at this capacity)
    assert (slot >= 0).all()
    key = ids.long() * C + slot.long()
    assert key.unique().numel() == key.numel()
    # gradients through the weights and through the probability sums (the auxiliary loss)
    gw = torch.randn(T, k, device="cuda")
    gp = torch.randn(E, device="cuda")
    (w * gw).sum().add((prob_sum * gp).sum()).backward()
    gw_ref = torch.zeros_like(gw).scatter(1, order[1], gw.gather(1, order[0]))     # same pairing as the kernel's order
    ((topw * gw_ref).sum() + (probs.sum(0) * gp).sum()).backward()
    got = logits.grad.float()
    assert torch.allclose(got[:, :E], lr.grad, atol=2e-2, rtol=2e-2), (got[:, :E] - lr.grad).abs().max()
    assert (got[:, E:] == 0).all()
    # a small capacity drops the late arrivals only
    _, _, ids2, slot2, _ = moe.route(logits.detach(), E, k, 8)
    for e in range(min(E, 4)):
        kept = (slot2[ids2 == e] >= 0).sum().item()
        assert kept == min(8, int((ids2 == e).sum()))
    # the slots are the arrival order by pair index (the same in every run): compare with the
    # index-ordered assignment written with PyTorch ops on the host
    ref_slot, ref_counts = moe.assign_slots(ids2.cpu(), E, 8)
    assert torch.equal(slot2.cpu(), ref_slot)
    ref_slot, ref_counts = moe.assign_slots(ids.cpu(), E, C)
    assert torch.equal(slot.cpu(), ref_slot) and torch.equal(counts.cpu(), ref_counts)


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (6, 5, 7, 9)), (torch.bfloat16, (8, 16, 33)),
                                         (torch.float32, (3, 64, 4, 4, 5))])
def test_batch_norm_kernels_match_the_pytorch_formulation(dtype, shape):
    """Per-feature sum, sum of squared deviations and the normalise + affine map (forward and backward)
    against the same expressions written with PyTorch operations in fp32."""
    from distdl_b200.ops import batchnorm as bn
    torch.manual_seed(3)
    F = shape[1]
    stat = (1, F) + (1,) * (len(shape) - 2)
    x = torch.randn(*shape, device="cuda").to(dtype).requires_grad_()
    mean = torch.randn(stat, device="cuda").mul(0.1).to(dtype).requires_grad_()
    var = (torch.rand(stat, device="cuda") + 0.5).to(dtype).requires_grad_()
    gamma = (1 + 0.1 * torch.randn(stat, device="cuda")).to(dtype).requires_grad_()
    beta = (0.1 * torch.randn(stat, device="cuda")).to(dtype).requires_grad_()
    dims = [d for d in range(len(shape)) if d != 1]
    tol = 1e-4 if dtype == torch.float32 else 3e-2

    def close(a, b):
        err = (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)
        assert err < tol, err

    ref = [t.detach().float().requires_grad_() for t in (x, mean, var, gamma, beta)]
    s, sr = bn.channel_sum(x), ref[0].sum(dims, keepdim=True)
    q, qr = bn.channel_sqdev(x, mean), ((ref[0] - ref[1]) ** 2).sum(dims, keepdim=True)
    y = bn.normalize(x, mean, var, gamma, beta, 1e-5)
    yr = ref[3] * (ref[0] - ref[1]) / torch.sqrt(ref[2] + 1e-5) + ref[4]
    close(s, sr)
    close(q, qr)
    close(y, yr)
    gs, gq, gy = torch.randn_like(sr), torch.randn_like(qr), torch.randn_like(yr)
    torch.autograd.backward([s, q, y], [gs.to(dtype), gq.to(dtype), gy.to(dtype)])
    torch.autograd.backward([sr, qr, yr], [gs.to(dtype).float(), gq.to(dtype).float(), gy.to(dtype).float()])
    for got, want in zip((x, mean, var, gamma, beta), ref):
        close(got.grad, want.grad)


@pytest.mark.parametrize("nd,kind,kernel,stride,dilation", [
    (1, "avg", (3,), (2,), (1,)), (1, "max", (3,), (1,), (2,)),
    (2, "avg", (2, 3), (2, 1), (1, 1)), (2, "max", (3, 3), (2, 2), (1, 1)), (2, "max", (2, 2), (1, 1), (2, 3)),
    (3, "avg", (2, 2, 2), (2, 2, 2), (1, 1, 1)), (3, "max", (3, 2, 3), (1, 2, 1), (1, 1, 2))])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pooling_kernels_match_torch_on_a_cropped_view(nd, kind, kernel, stride, dilation, dtype):
    import torch.nn.functional as F

    from distdl_b200.ops import pooling
    torch.manual_seed(3)
    space = {1: (37,), 2: (19, 23), 3: (9, 11, 13)}[nd]
    full = torch.randn(3, 5, *[n + 3 for n in space], device="cuda").to(dtype)
    crop = (slice(None), slice(None)) + tuple(slice(1, 1 + n) for n in space)
    x = full.clone().requires_grad_()
    xr = full.float().clone().requires_grad_()
    view = x[crop]
    assert pooling.usable(view) and not view.is_contiguous()
    y = pooling.pool(view, kind, kernel, stride, dilation)
    if kind == "avg":
        fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd]
        yr = fn(xr[crop], kernel, stride=stride)
    else:
        fn = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nd]
        yr = fn(xr[crop], kernel, stride=stride, dilation=dilation)
    assert y.shape == yr.shape
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert (y.float() - yr).abs().max().item() <= tol * (1 + yr.abs().max().item())
    dy = torch.randn_like(yr)
    y.backward(dy.to(dtype))
    yr.backward(dy)
    assert (x.grad.float() - xr.grad).abs().max().item() <= tol * (1 + xr.grad.abs().max().item()) * 4
