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
