"""Trains a small Llama-shaped decoder for a few steps on synthetic tokens with
tensor parallelism x ZeRO-3 (works on CPU ranks with gloo and on GPUs with the
native backend):

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/basics/train_decoder.py [--gpu]
"""
import sys

import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import say, start

P_world, rank = start(cpu="--gpu" not in sys.argv)
from distdl_b200 import models  # noqa: E402
from distdl_b200.parallel import SyntheticTokens, Trainer  # noqa: E402

world = P_world.size
tp = 2 if world % 2 == 0 else 1
layout = models.ParallelLayout(world // tp, tp, P_world)
on_gpu = "--gpu" in sys.argv
cfg = models.llama_tiny(dtype=torch.bfloat16 if on_gpu else torch.float32)
model = models.Decoder(cfg, layout)
local_batch, seq = 2, 256 if on_gpu else 64
trainer = Trainer(model, global_tokens_per_step=local_batch * layout.dp * seq, micro_batch=1, lr=3e-3, warmup_steps=2)
data = SyntheticTokens(local_batch, seq, cfg.vocab_size, dp_index=layout.dp_index)
block = data.next()
for step in range(10):
    loss = trainer.step(block).item()          # the same block every step: the loss must fall
    if rank == 0:
        print(f"step {step}: loss {loss:.4f}")
