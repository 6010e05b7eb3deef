"""A small decoder cut into two pipeline stages of two tensor-parallel workers each, trained by the
ordinary Trainer: the micro-batches of a step run through the one-forward-one-backward schedule.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/basics/ex_pipelined_decoder.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import say, start  # noqa: E402

P_world, rank = start()
from distdl_b200 import models  # noqa: E402
from distdl_b200.parallel import SyntheticTokens, Trainer  # noqa: E402

cfg = models.llama_tiny(dtype=torch.float32, n_layers=4)
torch.manual_seed(0)
piped = models.PipelinedDecoder(cfg, pp=2, dp=1, tp=P_world.size // 2)
local_batch, seq = 4, 64
trainer = Trainer(piped, global_tokens_per_step=local_batch * seq, micro_batch=1, lr=3e-3, warmup_steps=2)
block = SyntheticTokens(local_batch, seq, cfg.vocab_size).next()          # every process: the same block
say(P_world, "stage", piped.stage_index, "blocks", piped.model.layer_range,
    "parameters", sum(p.numel() for p in piped.parameters()))
for step in range(6):
    loss = trainer.step(block).item()
    if rank == 0:
        print(f"step {step}: loss {loss:.4f}")
