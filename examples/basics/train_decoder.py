"""Trains a small Llama-shaped decoder for a few steps on synthetic tokens with tensor parallelism x
ZeRO-3 (optionally context parallelism), saves a sharded checkpoint half-way, and resumes from it in
a fresh trainer.  Works on CPU ranks with gloo and on GPUs with the native backend:

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/basics/train_decoder.py [--gpu] [--cp 2]
"""
import os
import shutil
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import start  # noqa: E402

on_gpu = "--gpu" in sys.argv
cp = int(sys.argv[sys.argv.index("--cp") + 1]) if "--cp" in sys.argv else 1
P_world, rank = start(cpu=not on_gpu)
from distdl_b200 import models  # noqa: E402
from distdl_b200.parallel import Heartbeat, SyntheticTokens, Trainer  # noqa: E402

world = P_world.size
tp = 2 if (world // cp) % 2 == 0 else 1
cfg = models.llama_tiny(dtype=torch.bfloat16 if on_gpu else torch.float32)
local_batch, seq = 2, 256 if on_gpu else 64


def make_trainer():
    torch.manual_seed(0)
    layout = models.ParallelLayout(world // (tp * cp), tp, P_world, cp=cp)
    model = models.Decoder(cfg, layout)
    trainer = Trainer(model, global_tokens_per_step=local_batch * layout.dp * seq, micro_batch=1, lr=3e-3,
                      warmup_steps=2, heartbeat=heartbeat)
    return layout, trainer


heartbeat = Heartbeat(interval=1.0, limit=30.0).start()      # a silent rank raises RankFailure before a step
layout, trainer = make_trainer()
block = SyntheticTokens(local_batch, seq, cfg.vocab_size, dp_index=layout.dp_index).next()
folder = [tempfile.mkdtemp(prefix="distdl_ckpt_") if rank == 0 else None]
dist.broadcast_object_list(folder, src=0)
for step in range(10):
    loss = trainer.step(block).item()          # the same block every step: the loss must fall
    if rank == 0:
        print(f"step {step}: loss {loss:.4f}")
    if step == 4:
        trainer.save_checkpoint(folder[0])
# a fresh model and optimizer, as after a restart of the job: continue from step 5
_, resumed = make_trainer()
resumed.load_checkpoint(folder[0])
loss = resumed.step(block).item()
if rank == 0:
    print(f"resumed at step {resumed.steps_done - 1}: loss {loss:.4f} (matches step 5 above)")
heartbeat.leave()
dist.barrier()
if rank == 0:
    shutil.rmtree(folder[0], ignore_errors=True)
