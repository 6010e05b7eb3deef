"""The decoder models on CPU ranks: tensor parallel x ZeRO layouts train (the loss
falls on a repeated batch), uneven head splits work, all parameters get gradients."""
import math

import torch

from dist_harness import run_ranks


def body_train(rank, world, family, dp, tp, keep_gathered=False):
    from distdl_b200 import models
    from distdl_b200.parallel import SyntheticTokens, Trainer
    torch.manual_seed(0)
    cfg = {"llama": models.llama_tiny, "gpt2": models.gpt2_tiny}[family](dtype=torch.float32, max_seq=32,
                                                                       vocab_size=200, d_model=48, ffn_dim=96)
    if family == "gpt2":
        cfg.n_heads = cfg.n_kv_heads = 3          # 3 heads over 2 workers: 2 + 1
    else:
        cfg.n_heads, cfg.n_kv_heads = 4, 2
    cfg.keep_gathered = keep_gathered
    layout = models.ParallelLayout(dp, tp)
    model = models.Decoder(cfg, layout)
    trainer = Trainer(model, global_tokens_per_step=2 * dp * 32, micro_batch=1, lr=5e-3, warmup_steps=0,
                      max_grad_norm=1.0)
    data = SyntheticTokens(2, 32, cfg.vocab_size, dp_index=layout.dp_index)
    block = data.next()
    losses = [trainer.step(block).item() for _ in range(6)]
    assert all(math.isfinite(v) for v in losses), losses
    assert losses[-1] < losses[0] - 0.2, losses
    return losses


def test_llama_tp2_zero2_trains():
    out = run_ranks("test_models", "body_train", 4, args=("llama", 2, 2), timeout=300)
    assert out[0] == out[1] == out[2] == out[3]       # the all-reduced loss agrees everywhere


def test_gpt2_uneven_heads_tp2_trains():
    run_ranks("test_models", "body_train", 2, args=("gpt2", 1, 2), timeout=300)


def test_keep_gathered_matches_zero3():
    """Gathering once per step and reduce-scattering the gradients once gives the
    same training trajectory as re-gathering at every use."""
    a = run_ranks("test_models", "body_train", 4, args=("llama", 2, 2, False), timeout=300)[0]
    b = run_ranks("test_models", "body_train", 4, args=("llama", 2, 2, True), timeout=300)[0]
    for x, y in zip(a, b):
        assert abs(x - y) < 2e-4 * max(1.0, abs(x)), (a, b)


def body_trainer_checkpoint(rank, world, tmp):
    """save at step 3, keep training to step 6; a fresh trainer that loads the checkpoint
    reproduces steps 4-6 exactly; the metrics sink writes one JSON line per step on rank 0."""
    import json
    import os
    from distdl_b200 import models
    from distdl_b200.parallel import MetricsSink, SyntheticTokens, Trainer

    def make(metrics=None):
        torch.manual_seed(0)
        cfg = models.llama_tiny(dtype=torch.float32, max_seq=32, vocab_size=200, d_model=48, ffn_dim=96)
        cfg.n_heads, cfg.n_kv_heads = 4, 2
        layout = models.ParallelLayout(2, 1)
        model = models.Decoder(cfg, layout)
        return Trainer(model, global_tokens_per_step=2 * 2 * 32, micro_batch=1, lr=5e-3, warmup_steps=0,
                       metrics=metrics), layout, cfg

    sink = MetricsSink(os.path.join(tmp, "metrics.jsonl"))
    a, layout, cfg = make(sink)
    data = SyntheticTokens(2, 32, cfg.vocab_size, dp_index=layout.dp_index, seed=5, n_buffers=8)
    blocks = [data.next().clone() for _ in range(6)]
    for i in range(3):
        a.step(blocks[i])
    a.save_checkpoint(os.path.join(tmp, "ckpt"))
    ref = [a.step(blocks[i]).item() for i in range(3, 6)]
    sink.close()
    b, _, _ = make()
    manifest = b.load_checkpoint(os.path.join(tmp, "ckpt"))
    assert manifest["world_size"] == world and manifest["steps_done"] == 3 and manifest["layout"] == {"dp": 2, "tp": 1, "cp": 1}
    got = [b.step(blocks[i]).item() for i in range(3, 6)]
    assert all(abs(x - y) < 1e-6 * max(1.0, abs(x)) for x, y in zip(ref, got)), (ref, got)
    if rank == 0:
        lines = [json.loads(line) for line in open(os.path.join(tmp, "metrics.jsonl"))]
        assert [ln["step"] for ln in lines] == [1, 2, 3, 4, 5, 6] and all("loss" in ln for ln in lines)
    return True


def test_trainer_checkpoint_and_metrics(tmp_path):
    run_ranks("test_models", "body_trainer_checkpoint", 2, args=(str(tmp_path),), timeout=300)


def body_context_parallel(rank, world, family, tp):
    """Context parallelism (ring attention over two blocks of every sequence) against the same
    weights run WITHOUT it.  On the same worker grid, ``ParallelLayout(dp=1, cp=2, tp)`` and
    ``ParallelLayout(dp=2, cp=1, tp)`` shard every parameter identically, so the same seed gives the
    same model.  The data-parallel model is fed the whole sequences on both replicas: its summed
    loss and gradients are then exactly twice those of the context-parallel model, in which every
    worker sees one block and attention, rotary / learned positions and the token slicing have to
    reproduce the global sequence."""
    import torch.distributed as dist

    from distdl_b200 import models
    cfg = {"llama": models.llama_tiny, "gpt2": models.gpt2_tiny}[family](dtype=torch.float32, max_seq=32,
                                                                       vocab_size=200, d_model=48, ffn_dim=96)
    cfg.n_heads, cfg.n_kv_heads = (4, 2) if family == "llama" else (3, 3)
    cfg.n_layers = 2
    torch.manual_seed(0)
    cp_model = models.Decoder(cfg, models.ParallelLayout(1, tp, cp=2))
    torch.manual_seed(0)
    dp_model = models.Decoder(cfg, models.ParallelLayout(2, tp))
    for a, b in zip(cp_model.parameters(), dp_model.parameters()):
        assert a.shape == b.shape and torch.equal(a, b)
    gen = torch.Generator().manual_seed(5)
    tokens = torch.randint(0, cfg.vocab_size, (2, 33), generator=gen)        # the same on every worker
    out = {}
    for name, model in (("cp", cp_model), ("dp", dp_model)):
        model.train()
        loss = model.loss(tokens[:, :-1], tokens[:, 1:], scale=1.0 / 64)
        loss.backward()
        model.release_gathered()
        total = loss.detach().clone()
        dist.all_reduce(total)
        out[name] = (total, [None if p.grad is None else p.grad.clone() for p in model.parameters()])
    assert torch.allclose(out["cp"][0] * 2, out["dp"][0], rtol=1e-5), (out["cp"][0], out["dp"][0])
    names = [n for n, _ in cp_model.named_parameters()]
    for n, ga, gb in zip(names, out["cp"][1], out["dp"][1]):
        assert (ga is None) == (gb is None), n
        if ga is not None and ga.numel():
            assert torch.allclose(ga * 2, gb, rtol=2e-4, atol=2e-6), (n, (ga * 2 - gb).abs().max())
    return float(out["cp"][0])


def test_context_parallel_decoder_matches_full_sequence_attention():
    run_ranks("test_models", "body_context_parallel", 2, args=("llama", 1), timeout=300)
    run_ranks("test_models", "body_context_parallel", 4, args=("llama", 2), timeout=300)
    run_ranks("test_models", "body_context_parallel", 4, args=("gpt2", 2), timeout=300)
