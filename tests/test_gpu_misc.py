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
