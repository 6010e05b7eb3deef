"""Checkpoint / resume: per-rank sharded state (model + optimizer) resumes the
loss trajectory exactly; the collected serial-layout state moves a model between
world sizes (saved on a 2x2 grid, loaded on a 1x2 grid and on one worker)."""
import io

import torch

from dist_harness import run_ranks


def _mlp(P_feat, P_seq, collect):
    from distdl_b200.nn import DistributedLinearAllGatherZero, DistributedLinearReduceScatterZero

    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.up = DistributedLinearAllGatherZero(P_feat, 8, 16, P_x=P_seq, collect_state=collect)
            self.down = DistributedLinearReduceScatterZero(P_feat, 16, 8, P_y=P_seq, collect_state=collect)

        def forward(self, x):
            return self.down(torch.tanh(self.up(x)))
    return MLP()


def _parts(world):
    import distdl_b200 as d
    base = d.backends.backend.Partition().create_partition_inclusive(range(world))
    D = world // 2 if world >= 2 else 1
    M = 2 if world >= 2 else 1
    return base.create_cartesian_topology_partition([D, 1, M]), base.create_cartesian_topology_partition([D, M, 1])


def body_sharded_resume(rank, world):
    from distdl_b200.parallel import FlatAdamW
    torch.manual_seed(0)
    P_feat, P_seq = _parts(world)
    xs = [torch.randn(2, 4, 8, generator=torch.Generator().manual_seed(10 * s + rank)) for s in range(6)]

    def run(model, opt, steps):
        out = []
        for x in steps:
            loss = model(x).pow(2).sum()
            loss.backward()
            opt.step()
            out.append(round(loss.item(), 6))
        return out
    m = _mlp(P_feat, P_seq, False)
    opt = FlatAdamW(m, lr=1e-2, max_grad_norm=None)
    first = run(m, opt, xs[:3])
    buf = io.BytesIO()
    torch.save({"model": m.state_dict(), "opt": opt.state_dict()}, buf)      # one file per rank
    rest = run(m, opt, xs[3:])
    # resume in fresh objects from this rank's shard
    m2 = _mlp(P_feat, P_seq, False)
    opt2 = FlatAdamW(m2, lr=1e-2, max_grad_norm=None)
    buf.seek(0)
    ck = torch.load(buf, weights_only=False)
    m2.load_state_dict(ck["model"])
    opt2.load_state_dict(ck["opt"])
    rest2 = run(m2, opt2, xs[3:])
    assert rest == rest2, (rest, rest2)
    return first + rest


def test_sharded_checkpoint_resumes_loss_trajectory():
    run_ranks("test_checkpoint", "body_sharded_resume", 4, timeout=240)


def body_save_collected(rank, world):
    torch.manual_seed(0)
    P_feat, P_seq = _parts(world)
    m = _mlp(P_feat, P_seq, True)
    sd = m.state_dict()
    return {k: v.tolist() for k, v in sd.items()} if rank == 0 else None


def body_load_collected(rank, world, serial):
    from distdl_b200.nn import Repartition
    from distdl_b200.utilities.torch import zero_volume_tensor
    import distdl_b200 as d
    P_feat, P_seq = _parts(world)
    m = _mlp(P_feat, P_seq, True)
    sd = {k: (torch.tensor(v) if rank == 0 else zero_volume_tensor()) for k, v in serial.items()}
    m.load_state_dict(sd)
    # forward equals the serial model built from the same tensors
    xg = torch.randn(2, 4, 8, generator=torch.Generator().manual_seed(3))
    base = d.backends.backend.Partition().create_partition_inclusive(range(world))
    P_root = d.backends.backend.Partition().create_partition_inclusive([0]).create_cartesian_topology_partition([1, 1, 1])
    x = Repartition(P_root, P_seq, preserve_batch=False)(xg if rank == 0 else zero_volume_tensor())
    y = Repartition(P_seq, P_root, preserve_batch=False)(m(x))
    if rank == 0:
        W1, b1 = torch.tensor(serial["up.weight"]), torch.tensor(serial["up.bias"])
        W2, b2 = torch.tensor(serial["down.weight"]), torch.tensor(serial["down.bias"])
        ref = torch.nn.functional.linear(torch.tanh(torch.nn.functional.linear(xg, W1, b1)), W2, b2)
        assert torch.allclose(y, ref, atol=1e-5), (y - ref).abs().max()
    return True


def test_collected_checkpoint_moves_between_world_sizes():
    serial = run_ranks("test_checkpoint", "body_save_collected", 4, timeout=240)[0]
    assert set(serial) == {"up.weight", "up.bias", "down.weight", "down.bias"}
    assert torch.tensor(serial["up.weight"]).shape == (16, 8)
    run_ranks("test_checkpoint", "body_load_collected", 2, args=(serial,), timeout=240)
    run_ranks("test_checkpoint", "body_load_collected", 1, args=(serial,), timeout=240)
