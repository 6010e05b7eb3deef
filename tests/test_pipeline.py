"""1F1B pipeline over CPU ranks against the serial model: same loss, same gradients."""
import torch

from dist_harness import run_ranks


def _layers(n_stages, width=16):
    torch.manual_seed(3)
    return [torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.Tanh()) for _ in range(n_stages)]


def body_pipeline(rank, world, n_micro):
    from distdl_b200.parallel import PipelineStage, run_1f1b
    layers = _layers(world)
    torch.manual_seed(7)
    xs = [torch.randn(4, 16) for _ in range(n_micro)]
    ts = [torch.randn(4, 16) for _ in range(n_micro)]
    loss_fn = lambda y, t: ((y - t) ** 2).mean()      # noqa: E731
    # serial reference
    ref = _layers(world)
    ref_loss = 0.0
    for x, t in zip(xs, ts):
        h = x
        for layer in ref:
            h = layer(h)
        loss = loss_fn(h, t)
        loss.backward()
        ref_loss += loss.item()
    # pipeline: this rank owns layer `rank`
    stage = PipelineStage(layers[rank], list(range(world)), act_shape=(4, 16))
    total = run_1f1b(stage, xs if stage.first else None, ts if stage.last else None, loss_fn, n_micro=n_micro)
    if stage.last:
        assert abs(total.item() - ref_loss) < 1e-5, (total.item(), ref_loss)
    for p, q in zip(layers[rank].parameters(), ref[rank].parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6), (p.grad - q.grad).abs().max()
    return True


def test_1f1b_two_stages():
    run_ranks("test_pipeline", "body_pipeline", 2, args=(5,), timeout=120)


def test_1f1b_three_stages_fewer_micro_batches_than_stages():
    run_ranks("test_pipeline", "body_pipeline", 3, args=(2,), timeout=120)
    run_ranks("test_pipeline", "body_pipeline", 3, args=(6,), timeout=120)
