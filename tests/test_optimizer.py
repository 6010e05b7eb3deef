"""FlatAdamW on CPU ranks: identical slot layout on all workers (also when a worker holds a
zero-size shard of a parameter), update equal to torch.optim.AdamW, gradient clipping by
the global norm."""
import torch

from dist_harness import run_ranks


def body_flat_adamw(rank, world):
    import torch.distributed as dist
    from distdl_b200.parallel import FlatAdamW

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(3)
            a = torch.randn(5)
            self.a = torch.nn.Parameter(a if rank == 0 else torch.zeros(0))      # lives on worker 0 only
            self.b = torch.nn.Parameter(torch.randn(8) + rank)

    m, ref = M(), M()
    opt = FlatAdamW(m, lr=1e-2, weight_decay=0.1, max_grad_norm=None, no_decay=())
    totals = [None] * world
    dist.all_gather_object(totals, (opt.total, opt.uniform_layout))
    assert all(t == totals[0] for t in totals) and totals[0][1], totals      # same layout everywhere
    tref = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(3):
        for mod in (m, ref):
            loss = (mod.b ** 2).sum() + (mod.a ** 3).sum()
            loss.backward()
        opt.step()
        tref.step()
        tref.zero_grad()
        assert torch.allclose(m.b, ref.b, atol=1e-5), (step, (m.b - ref.b).abs().max())
        if rank == 0:
            assert torch.allclose(m.a, ref.a, atol=1e-5)
    return True


def body_clip(rank, world):
    import torch.distributed as dist
    from distdl_b200.parallel import FlatAdamW
    torch.manual_seed(rank)
    lin = torch.nn.Linear(4, 4)
    opt = FlatAdamW(lin, lr=1e-2, max_grad_norm=0.5)
    lin(torch.randn(3, 4)).pow(2).sum().backward()
    local_sq = opt.grad.pow(2).sum()
    dist.all_reduce(local_sq)
    opt.step()
    assert abs(float(opt.last_grad_norm) - float(local_sq.sqrt())) < 1e-5
    return True


def body_rank_without_parameters(rank, world):
    """An inactive worker (no trainable parameter at all) must still pass through every collective
    step of the optimizer's constructor and of step(), or the other workers block."""
    from distdl_b200.parallel import FlatAdamW

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(5)
            if rank != world - 1:                       # the last worker holds nothing
                self.w = torch.nn.Parameter(torch.randn(6) + rank)

    for clip in (None, 1.0):
        m, ref = M(), M()
        opt = FlatAdamW(m, lr=1e-2, weight_decay=0.0, max_grad_norm=clip, no_decay=())
        assert (opt.total == 0) == (rank == world - 1)
        tref = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0) \
            if rank != world - 1 else None
        for _ in range(2):
            if rank != world - 1:
                (m.w ** 2).sum().mul(1e-3).backward()
                (ref.w ** 2).sum().mul(1e-3).backward()
            opt.step()
            if tref is not None:
                tref.step()
                tref.zero_grad()
                assert torch.allclose(m.w, ref.w, atol=1e-5)        # (the small gradient is never clipped)
        opt.zero_grad()
    return True


def test_flat_adamw_matches_torch_and_layout_is_uniform():
    run_ranks("test_optimizer", "body_flat_adamw", 2, timeout=120)


def test_global_gradient_norm():
    run_ranks("test_optimizer", "body_clip", 2, timeout=120)


def test_worker_without_parameters_joins_every_collective_step():
    run_ranks("test_optimizer", "body_rank_without_parameters", 3, timeout=120)
