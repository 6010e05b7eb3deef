"""Memory-bound kernels against plain fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    assert err / scale < tol, f"err {err} scale {scale}"


@pytest.mark.parametrize("d", [1024, 1600, 4096])
@pytest.mark.parametrize("rms", [True, False])
def test_norm_fwd_bwd(d, rms):
    from distdl_b200.ops import layer_norm, rms_norm
    torch.manual_seed(0)
    rows = 777
    x = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_()
    b = None if rms else (0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = rms_norm(x, w, 1e-5) if rms else layer_norm(x, w, b, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    else:
        br = b.detach().float().requires_grad_()
        yr = torch.nn.functional.layer_norm(xr, (d,), wr, br, 1e-5)
    yr.backward(dy.float())
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(w.grad, wr.grad)
    if not rms:
        _close(b.grad, br.grad)


@pytest.mark.parametrize("rms", [True, False])
def test_add_norm_returns_sum_and_norm_with_the_gradient_of_both(rms):
    """The residual add fused into the norm: both outputs and, in backward, gradients arriving on both."""
    from distdl_b200.ops import add_layer_norm, add_rms_norm
    torch.manual_seed(1)
    rows, d = 515, 4096
    x = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_()
    b = None if rms else (0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_()
    s, y = add_rms_norm(x, r, w, 1e-5) if rms else add_layer_norm(x, r, w, b, 1e-5)
    ds, dy = torch.randn_like(s), torch.randn_like(y)
    torch.autograd.backward([s, y], [ds, dy])
    xr, rr = x.detach().float().requires_grad_(), r.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    sr = (xr + rr).detach().to(torch.bfloat16).float() + (xr + rr - (xr + rr).detach())     # the stored sum is bf16
    if rms:
        yr = sr * torch.rsqrt(sr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    else:
        br = b.detach().float().requires_grad_()
        yr = torch.nn.functional.layer_norm(sr, (d,), wr, br, 1e-5)
    torch.autograd.backward([sr, yr], [ds.float(), dy.float()])
    _close(s, sr)
    _close(y, yr)
    _close(x.grad, xr.grad)
    _close(r.grad, rr.grad)
    _close(w.grad, wr.grad)
    # only the sum is used downstream: the gradient passes through untouched
    x2 = x.detach().requires_grad_()
    s2, _ = add_rms_norm(x2, r.detach(), w.detach(), 1e-5)
    s2.backward(ds)
    assert torch.equal(x2.grad, ds)


def test_rope_on_the_projection_output_rotates_in_place_without_copying_gradients():
    from distdl_b200.ops import rope_
    torch.manual_seed(0)
    b, seq, hq, hk, hd = 2, 64, 4, 2, 128
    lin = torch.randn(b, seq, (hq + 2 * hk) * hd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = lin * 1.0                                                     # a non-leaf, like a projection's output
    ref = rope_(y.detach().clone().reshape(b * seq, hq + 2 * hk, hd), seq, hq + hk, theta=10000.0)
    out = rope_(y, seq, hq + hk, theta=10000.0, layout=(b * seq, hq + 2 * hk, hd))
    assert out.shape == lin.shape and torch.equal(out.reshape(ref.shape), ref)
    g = torch.randn_like(out)
    out.backward(g.clone())           # the node rotates the gradient it is handed in place
    # the adjoint of a rotation is the inverse rotation: rotating the gradient forward again gives g
    back = rope_(lin.grad.clone().reshape(b * seq, hq + 2 * hk, hd), seq, hq + hk, theta=10000.0)
    _close(back, g.reshape(back.shape), 1e-2)


def test_swiglu_gelu():
    from distdl_b200.ops import gelu, swiglu
    torch.manual_seed(0)
    gu = torch.randn(300, 2 * 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = swiglu(gu)
    dy = torch.randn_like(y)
    y.backward(dy)
    r = gu.detach().float().requires_grad_()
    yr = torch.nn.functional.silu(r[:, :512]) * r[:, 512:]
    yr.backward(dy.float())
    _close(y, yr)
    _close(gu.grad, r.grad)
    x = torch.randn(300, 640, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = gelu(x)
    y.backward(dy[:, :1].expand(300, 640).contiguous())
    r = x.detach().float().requires_grad_()
    yr = torch.nn.functional.gelu(r, approximate="tanh")
    yr.backward(dy[:, :1].expand(300, 640).float())
    _close(y, yr)
    _close(x.grad, r.grad)


def test_rope_roundtrip_and_reference():
    from distdl_b200.ops import rope_, rope_table
    torch.manual_seed(0)
    seq, hq, hk, hd = 64, 4, 2, 128
    tokens = 2 * seq
    qkv = torch.randn(tokens, hq + 2 * hk, hd, device="cuda", dtype=torch.bfloat16)
    ref_in = qkv.clone()
    out = rope_(qkv.clone(), seq, hq + hk, theta=10000.0)
    table = rope_table(seq, hd, 10000.0, qkv.device)
    pos = torch.arange(tokens, device="cuda") % seq
    cos = table[pos, :, 0].unsqueeze(1)
    sin = table[pos, :, 1].unsqueeze(1)
    x = ref_in[:, : hq + hk].float()
    a, b = x[..., : hd // 2], x[..., hd // 2:]
    ref = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    _close(out[:, : hq + hk], ref)
    assert torch.equal(out[:, hq + hk:], ref_in[:, hq + hk:])


def test_embedding_and_xent():
    from distdl_b200.ops import cross_entropy_, embedding
    torch.manual_seed(0)
    V, d, T = 1000, 256, 333
    table = torch.randn(V, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, V, (T,), device="cuda")
    e = embedding(ids, table)
    assert torch.equal(e, table.detach()[ids])
    g = torch.randn_like(e)
    e.backward(g)
    ref = torch.zeros(V, d, device="cuda")
    ref.index_add_(0, ids, g.float())
    _close(table.grad, ref)

    ld = 1008
    logits = torch.randn(T, ld, device="cuda", dtype=torch.bfloat16)
    lr = logits[:, :V].detach().float().requires_grad_()
    tgt = torch.randint(0, V, (T,), device="cuda")
    loss_ref = torch.nn.functional.cross_entropy(lr, tgt)
    loss_ref.backward()
    lg = logits.clone().requires_grad_()
    work = lg * 1  # non-leaf that the op may overwrite
    loss = cross_entropy_(work, tgt, vocab=V, unit_grad=True)
    loss.backward()
    assert abs(loss.item() - loss_ref.item()) < 2e-2
    _close(lg.grad[:, :V], lr.grad, tol=3e-2)
    assert lg.grad[:, V:].abs().max().item() == 0


def test_adamw_matches_torch():
    from distdl_b200.ops import adamw_step_, sumsq_
    torch.manual_seed(0)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    master = p.clone()
    for step in range(1, 4):
        ref.grad = g.clone()
        opt.step()
        gg = g.clone()
        adamw_step_(master, m, v, gg, pb, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
        assert gg.abs().max().item() == 0
    assert (master - ref.detach()).abs().max().item() < 1e-5
    _close(pb, master)
    out = torch.zeros(1, device="cuda")
    sumsq_(g, out)
    assert abs(out.item() - (g.double() ** 2).sum().item()) / n < 1e-3


def test_accumulate_into_fp32_buffer():
    """acc(fp32) += scale * g(bf16): the cast-and-add kernel of the gradient accumulators."""
    from distdl_b200.ops.optim import accumulate_f32_
    torch.manual_seed(2)
    n = 1 << 20
    acc = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").to(torch.bfloat16)
    want = acc + 0.5 * g.float()
    accumulate_f32_(acc, g, 0.5)
    assert torch.allclose(acc, want, atol=1e-6)
    g32 = torch.randn(1000, device="cuda")                # other dtypes take the PyTorch path
    acc2 = torch.zeros(1000, device="cuda")
    accumulate_f32_(acc2, g32)
    assert torch.equal(acc2, g32)
