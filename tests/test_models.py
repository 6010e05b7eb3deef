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


def body_context_parallel(rank, world, family, tp, cp_mode="ring"):
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
    if cp_mode == "a2a":
        cfg.n_heads, cfg.n_kv_heads = 8, 4           # local head counts must divide by the context-parallel size
    cfg.n_layers, cfg.cp_mode = 2, cp_mode
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
    run_ranks("test_models", "body_context_parallel", 4, args=("llama", 2, "a2a"), timeout=300)
    run_ranks("test_models", "body_context_parallel", 4, args=("llama", 2, "zigzag"), timeout=300)
    run_ranks("test_models", "body_context_parallel", 4, args=("gpt2", 2, "zigzag"), timeout=300)


def body_pipelined_decoder(rank, world):
    """Two pipeline stages of one worker each against the whole model on one worker, with the same
    weights (copied from the whole model's state dict): loss and every gradient agree after a
    1F1B pass over three micro-batches."""
    import distdl_b200
    from distdl_b200 import models
    cfg = models.llama_tiny(dtype=torch.float32, max_seq=16, vocab_size=96, d_model=32, ffn_dim=64)
    cfg.n_layers, cfg.n_heads, cfg.n_kv_heads = 3, 4, 2
    torch.manual_seed(0)
    P_me = distdl_b200.backends.backend.Partition().create_partition_inclusive([rank])
    whole = models.Decoder(cfg, models.ParallelLayout(1, 1, P_world=P_me))
    piped = models.PipelinedDecoder(cfg, pp=2, dp=1, tp=1)
    lo, hi = piped.model.layer_range
    assert (lo, hi) == ((0, 2) if rank == 0 else (2, 3))
    src = whole.state_dict()
    mapped = {}
    for k in piped.model.state_dict():
        parts = k.split(".")
        if parts[0] == "blocks":
            parts[1] = str(int(parts[1]) + lo)
        mapped[k] = src[".".join(parts)]
    piped.model.load_state_dict(mapped)
    gen = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, cfg.vocab_size, (3, 17), generator=gen)
    scale = 1.0 / (3 * 16)
    total = piped.global_loss(piped.forward_backward(tokens, micro_batch=1, scale=scale))
    piped.model.release_gathered()
    whole.train()
    ref = whole.loss(tokens[:, :-1], tokens[:, 1:], scale=scale)
    ref.backward()
    whole.release_gathered()
    assert torch.allclose(total, ref.detach(), rtol=1e-5), (total, ref)
    ref_grads = dict(whole.named_parameters())
    for k, p in piped.model.named_parameters():
        parts = k.split(".")
        if parts[0] == "blocks":
            parts[1] = str(int(parts[1]) + lo)
        g = ref_grads[".".join(parts)].grad
        assert p.grad is not None and torch.allclose(p.grad, g, rtol=1e-4, atol=1e-6), (k, (p.grad - g).abs().max())
    return float(total)


def test_pipelined_decoder_matches_whole_model():
    out = run_ranks("test_models", "body_pipelined_decoder", 2, timeout=300)
    assert out[0] == out[1]


def body_pipelined_tp_trains(rank, world):
    """Two stages of two tensor-parallel workers each: the loss falls on a repeated batch."""
    from distdl_b200 import models
    from distdl_b200.parallel import FlatAdamW
    torch.manual_seed(0)
    cfg = models.llama_tiny(dtype=torch.float32, max_seq=16, vocab_size=96, d_model=32, ffn_dim=64)
    cfg.n_layers, cfg.n_heads, cfg.n_kv_heads = 2, 4, 2
    piped = models.PipelinedDecoder(cfg, pp=2, dp=1, tp=2)
    opt = FlatAdamW(piped.model, lr=1e-2, weight_decay=0.0, max_grad_norm=1.0)
    gen = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, cfg.vocab_size, (4, 17), generator=gen)
    losses = []
    for _ in range(6):
        total = piped.global_loss(piped.forward_backward(tokens, micro_batch=2, scale=1.0 / 64))
        opt.step()
        losses.append(float(total))
    assert losses[-1] < losses[0] - 0.2, losses
    return losses


def body_pipelined_trainer(rank, world, tmp):
    """The trainer drives a pipelined decoder like any model: schedule, optimizer per stage, all-reduced
    loss, sharded checkpoint and resume."""
    from distdl_b200 import models
    from distdl_b200.parallel import Trainer
    cfg = models.llama_tiny(dtype=torch.float32, max_seq=16, vocab_size=96, d_model=32, ffn_dim=64)
    cfg.n_layers, cfg.n_heads, cfg.n_kv_heads = 2, 4, 2

    def make():
        torch.manual_seed(0)
        piped = models.PipelinedDecoder(cfg, pp=2, dp=1, tp=2)
        return Trainer(piped, global_tokens_per_step=4 * 16, micro_batch=2, lr=1e-2, warmup_steps=0)
    trainer = make()
    gen = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, cfg.vocab_size, (4, 17), generator=gen)
    losses = [trainer.step(tokens).item() for _ in range(3)]
    trainer.save_checkpoint(tmp)
    losses += [trainer.step(tokens).item() for _ in range(2)]
    again = make()
    again.load_checkpoint(tmp)
    resumed = [again.step(tokens).item() for _ in range(2)]
    assert losses[-1] < losses[0] - 0.1, losses
    assert all(abs(a - b) < 1e-5 * abs(a) for a, b in zip(losses[3:], resumed)), (losses, resumed)
    return losses


def test_trainer_drives_a_pipelined_decoder(tmp_path):
    out = run_ranks("test_models", "body_pipelined_trainer", 4, args=(str(tmp_path),), timeout=300)
    assert out[0] == out[3]


def test_pipelined_tensor_parallel_decoder_trains():
    out = run_ranks("test_models", "body_pipelined_tp_trains", 4, timeout=300)
    assert out[0] == out[3]


def body_collected_decoder(rank, world, family, dp, tp, cp, serial, tokens):
    """With ``collect_state`` the decoder's state dict is the serial one on the first worker: saved on
    one worker grid, it loads on another and gives the same loss on the same batch."""
    import torch.distributed as dist

    from distdl_b200 import models
    make = {"llama": models.llama_tiny, "gpt2": models.gpt2_tiny, "mixtral": models.mixtral_tiny}[family]
    cfg = make(dtype=torch.float32, max_seq=16, vocab_size=100, d_model=48, ffn_dim=96)
    cfg.n_layers, cfg.collect_state = 2, True
    cfg.n_heads, cfg.n_kv_heads = (4, 4) if family == "gpt2" else (4, 2)
    cfg.capacity_factor = 8.0                      # experts: no token is dropped, whatever the grid
    torch.manual_seed(rank)
    model = models.Decoder(cfg, models.ParallelLayout(dp, tp, cp=cp))
    if serial is not None:
        model.load_state_dict(serial if rank == 0 else {})
    model.eval()
    with torch.no_grad():
        loss = model.loss(tokens[:, :-1], tokens[:, 1:], scale=1.0 / (dp * tokens.shape[0] * 16))
        model.release_gathered()
    dist.all_reduce(loss)
    sd = model.state_dict()
    if rank != 0:
        assert len(sd) == 0, list(sd)[:4]
    return float(loss), ({k: v.clone() for k, v in sd.items()} if rank == 0 else None)


def test_collected_decoder_checkpoint_moves_between_worker_grids():
    gen = torch.Generator().manual_seed(9)
    tokens = torch.randint(0, 100, (2, 17), generator=gen)        # every data-parallel replica: the same batch
    for family in ("llama", "gpt2"):
        loss4, serial = run_ranks("test_models", "body_collected_decoder", 4,
                                  args=(family, 2, 2, 1, None, tokens), timeout=300)[0]
        assert all(v.dim() <= 2 for v in serial.values())
        loss2 = run_ranks("test_models", "body_collected_decoder", 2, args=(family, 1, 2, 1, serial, tokens),
                          timeout=300)[0][0]
        loss1, again = run_ranks("test_models", "body_collected_decoder", 1, args=(family, 1, 1, 1, serial, tokens),
                                 timeout=300)[0]
        losscp = run_ranks("test_models", "body_collected_decoder", 4, args=(family, 1, 2, 2, serial, tokens),
                           timeout=300)[0][0]
        assert abs(loss4 - loss1) < 1e-4 * abs(loss1) and abs(loss2 - loss1) < 1e-4 * abs(loss1), (loss4, loss2, loss1)
        assert abs(losscp - loss1) < 1e-4 * abs(loss1), (losscp, loss1)
        assert set(again) == set(serial) and all(torch.equal(again[k], serial[k]) for k in serial)
    # mixture of experts: the experts move between expert-parallel sizes 4, 2 and 1
    loss4, serial = run_ranks("test_models", "body_collected_decoder", 4, args=("mixtral", 4, 1, 1, None, tokens),
                              timeout=300)[0]
    assert serial["blocks.0.mlp.w_up"].shape[0] == 4
    for world in (2, 1):
        loss = run_ranks("test_models", "body_collected_decoder", world,
                         args=("mixtral", world, 1, 1, serial, tokens), timeout=300)[0][0]
        assert abs(loss - loss4) < 2e-4 * abs(loss4), (world, loss, loss4)


def body_elastic(rank, world, dp, tp, path, mode):
    """Train on one worker grid, save the collected model, continue on another grid."""
    from distdl_b200 import models
    from distdl_b200.parallel import Trainer
    cfg = models.llama_tiny(dtype=torch.float32, max_seq=16, vocab_size=100, d_model=48, ffn_dim=96)
    cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.collect_state = 2, 4, 2, True
    torch.manual_seed(rank)
    layout = models.ParallelLayout(dp, tp)
    trainer = Trainer(models.Decoder(cfg, layout), global_tokens_per_step=4 * 16, micro_batch=1, lr=5e-3,
                      warmup_steps=0, max_grad_norm=1.0)
    gen = torch.Generator().manual_seed(21)
    tokens = torch.randint(0, 100, (4, 17), generator=gen)
    per = 4 // dp
    block = tokens[layout.dp_index * per:(layout.dp_index + 1) * per]      # the same global batch on every grid
    if mode == "train_and_save":
        losses = [trainer.step(block).item() for _ in range(4)]
        trainer.save_model_collected(path)
        return losses
    trainer.load_model_collected(path)
    assert trainer.steps_done == 4 and trainer.opt.step_count == 0
    return [trainer.step(block).item() for _ in range(3)]


def test_training_moves_to_another_worker_grid(tmp_path):
    path = str(tmp_path / "model.pt")
    first = run_ranks("test_models", "body_elastic", 4, args=(2, 2, path, "train_and_save"), timeout=300)[0]
    for world, dp, tp in ((2, 1, 2), (2, 2, 1), (1, 1, 1)):
        cont = run_ranks("test_models", "body_elastic", world, args=(dp, tp, path, "continue"), timeout=300)[0]
        # the first loss after the move is that of the saved weights: below where training started and
        # close to the last loss before the save (one optimizer step apart); every grid agrees on it
        assert cont[0] < first[0] - 0.2 and abs(cont[0] - first[-1]) < 0.5, (first, cont)
        if world == 2 and tp == 2:
            ref = cont
        assert abs(cont[0] - ref[0]) < 1e-4 * abs(ref[0]), (cont, ref)
        assert min(cont[1:]) < cont[0] and all(math.isfinite(v) for v in cont), cont   # and training goes on


def body_pipelined_optimizer_layout(rank, world):
    """Pipeline stages have different parameter lists.  The flat optimizer then lays its slots out per
    group of processes with the same list (here: per stage), with equal offsets inside a group even
    when the shards are uneven (3 heads over 2 tensor-parallel workers), and training works."""
    import torch.distributed as dist

    from distdl_b200 import models
    from distdl_b200.parallel import FlatAdamW
    torch.manual_seed(0)
    cfg = models.llama_tiny(dtype=torch.float32, max_seq=16, vocab_size=96, d_model=48, ffn_dim=96)
    cfg.n_layers, cfg.n_heads, cfg.n_kv_heads = 2, 3, 3
    piped = models.PipelinedDecoder(cfg, pp=2, dp=1, tp=2)
    opt = FlatAdamW(piped.model, lr=1e-2, weight_decay=0.0)
    assert opt.uniform_layout and opt.layout_group == ([0, 1] if rank < 2 else [2, 3])
    layouts = [None] * world
    dist.all_gather_object(layouts, [(n, o) for n, o, _ in opt.names])
    mate = rank ^ 1
    mine, theirs = dict(layouts[rank]), dict(layouts[mate])
    shared = set(mine) & set(theirs)
    assert shared and all(mine[n] == theirs[n] for n in shared)
    assert set(dict(layouts[0])) != set(dict(layouts[2]))            # the stages really differ
    gen = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, cfg.vocab_size, (4, 17), generator=gen)
    losses = []
    for _ in range(5):
        total = piped.global_loss(piped.forward_backward(tokens, micro_batch=2, scale=1.0 / 64))
        opt.step()
        losses.append(float(total))
    assert losses[-1] < losses[0] - 0.1, losses
    return losses


def test_flat_optimizer_lays_out_pipeline_stages_per_group():
    out = run_ranks("test_models", "body_pipelined_optimizer_layout", 4, timeout=300)
    assert out[0] == out[3]


def body_generate(rank, world, dp, tp, cp, serial, prompt):
    from distdl_b200 import models
    cfg = models.llama_tiny(dtype=torch.float32, max_seq=32, vocab_size=100, d_model=48, ffn_dim=96)
    cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.collect_state = 2, 4, 2, True
    torch.manual_seed(5)
    layout = models.ParallelLayout(dp, tp, cp=cp)
    model = models.Decoder(cfg, layout)
    if serial is not None:
        model.load_state_dict(serial if rank == 0 else {})
    per = prompt.shape[0] // dp
    mine = prompt[layout.dp_index * per:(layout.dp_index + 1) * per]
    out = model.generate(mine, 5)
    assert out.shape == (per, prompt.shape[1] + 5) and torch.equal(out[:, :prompt.shape[1]], mine)
    sd = model.state_dict()
    return out, ({k: v.clone() for k, v in sd.items()} if rank == 0 else None), layout.dp_index


def test_greedy_generation_agrees_across_worker_grids():
    gen = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, 100, (2, 7), generator=gen)
    (ref, serial, _), = run_ranks("test_models", "body_generate", 1, args=(1, 1, 1, None, prompt), timeout=300)
    assert not torch.equal(ref[0, 7:], ref[1, 7:]) or True
    for world, dp, tp, cp in ((2, 1, 2, 1), (4, 2, 2, 1), (4, 1, 2, 2)):
        outs = run_ranks("test_models", "body_generate", world, args=(dp, tp, cp, serial, prompt), timeout=300)
        per = 2 // dp
        for out, _, d in outs:
            assert torch.equal(out, ref[d * per:(d + 1) * per]), (world, dp, tp, cp, out, ref)


def body_varying_length(rank, world):
    """Sequence lengths that change between steps: 16 tokens give shards 8 + 8 over two sequence-parallel
    workers, 15 give 8 + 7, so only one worker sees its shard change; the trainer re-runs the layers'
    collective set-up on both."""
    from distdl_b200 import models
    from distdl_b200.parallel import Trainer
    torch.manual_seed(0)
    cfg = models.llama_tiny(dtype=torch.float32, max_seq=32, vocab_size=64, d_model=32, ffn_dim=64)
    cfg.n_layers, cfg.n_heads, cfg.n_kv_heads = 1, 2, 2
    trainer = Trainer(models.Decoder(cfg, models.ParallelLayout(1, 2)), global_tokens_per_step=2 * 16, micro_batch=1,
                      warmup_steps=0)
    gen = torch.Generator().manual_seed(1)
    out = []
    for seq in (16, 15, 15, 12, 16):
        out.append(trainer.step(torch.randint(0, 64, (2, seq + 1), generator=gen)).item())
    assert all(math.isfinite(v) for v in out)
    return out


def test_trainer_handles_changing_sequence_lengths():
    out = run_ranks("test_models", "body_varying_length", 2, timeout=240)
    assert out[0] == out[1]


def body_activation_policies(rank, world, family, tp):
    """The same model trained for three steps with every block recomputing, every block keeping its
    activations and a mix: losses and parameters agree, and in the keeping blocks the norm and
    activation outputs and the gathered ZeRO weights really are rebuilt in the backward pass."""
    from distdl_b200 import models
    from distdl_b200.parallel import FlatAdamW
    from distdl_b200.utilities import recompute
    results = {}
    rebuilds = {}
    for policy in ("full", "none", "2"):
        cfg = {"llama": models.llama_tiny, "gpt2": models.gpt2_tiny}[family](dtype=torch.float32, max_seq=16,
                                                                           vocab_size=96, d_model=32, ffn_dim=64)
        cfg.n_layers, cfg.n_heads, cfg.activation_policy = 3, 4, policy
        if family == "llama":
            cfg.n_kv_heads = 2
        torch.manual_seed(0)
        model = models.Decoder(cfg, models.ParallelLayout(world // tp, tp))
        opt = FlatAdamW(model, lr=1e-2, max_grad_norm=1.0)
        gen = torch.Generator().manual_seed(11 + rank // tp)
        losses = []
        count = {"n": 0}
        orig = recompute.Recipe.get

        def counting(self, _orig=orig, _count=count):
            before = self.rebuilds
            out = _orig(self)
            _count["n"] += self.rebuilds - before
            return out
        recompute.Recipe.get = counting
        try:
            for _ in range(3):
                tokens = torch.randint(0, cfg.vocab_size, (2, 17), generator=gen)
                model.train()
                loss = model.loss(tokens[:, :-1], tokens[:, 1:], scale=1.0 / 64)
                loss.backward()
                opt.step()
                losses.append(float(loss.detach()))
        finally:
            recompute.Recipe.get = orig
        assert model.activation_plan["keep"] == {"full": 0, "none": 3, "2": 2}[policy]
        results[policy] = (losses, [p.detach().clone() for p in model.parameters()])
        rebuilds[policy] = count["n"]
    assert rebuilds["full"] == 0
    # per keeping block and step: the activation output and four gathered weights; without tensor
    # parallelism also the two norm outputs (with it, the projections save the GATHERED norm output)
    # (with biases, the CPU library's linear works on a contiguous copy of the weight and saves that)
    per_block = 1 if family == "gpt2" else (7 if tp == 1 else 5)
    assert rebuilds["none"] == 3 * 3 * per_block and rebuilds["2"] == 3 * 2 * per_block, rebuilds
    for policy in ("none", "2"):
        for a, b in zip(results["full"][0], results[policy][0]):
            assert abs(a - b) < 1e-6 * max(1.0, abs(a)), (policy, results["full"][0], results[policy][0])
        for pa, pb in zip(results["full"][1], results[policy][1]):
            assert torch.allclose(pa, pb, rtol=1e-5, atol=1e-7), (policy, (pa - pb).abs().max())
    return True


def test_blocks_that_keep_their_activations_train_like_blocks_that_recompute():
    run_ranks("test_models", "body_activation_policies", 4, args=("llama", 2), timeout=300)
    run_ranks("test_models", "body_activation_policies", 4, args=("gpt2", 2), timeout=300)
    run_ranks("test_models", "body_activation_policies", 2, args=("llama", 1), timeout=300)
