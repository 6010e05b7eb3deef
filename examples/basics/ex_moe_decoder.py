"""A small mixture-of-experts decoder trained with expert parallelism: every worker owns one expert
of each block (top-2 routing over 4 experts), attention / router / embedding weights are ZeRO-sharded
over the same workers.  Shows the routing statistics of the first block next to the loss.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/basics/ex_moe_decoder.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import say, start  # noqa: E402

P_world, rank = start()
from distdl_b200 import models  # noqa: E402
from distdl_b200.ops import moe as moe_ops  # noqa: E402
from distdl_b200.parallel import SyntheticTokens, Trainer  # noqa: E402

cfg = models.mixtral_tiny(dtype=torch.float32, n_experts=P_world.size, d_model=64, ffn_dim=96, n_heads=2,
                          n_kv_heads=1, vocab_size=200, max_seq=32)
torch.manual_seed(0)
model = models.Decoder(cfg, models.ParallelLayout(P_world.size, 1))         # expert parallel over all workers
local_batch, seq = 4, 32
trainer = Trainer(model, global_tokens_per_step=P_world.size * local_batch * seq, micro_batch=2, lr=3e-3,
                  warmup_steps=2)
block = SyntheticTokens(local_batch, seq, cfg.vocab_size, seed=10 + rank).next()     # one block per worker, reused
say(P_world, "local experts", model.blocks[0].mlp.w_up.shape[0], "of", cfg.n_experts,
    "parameters", sum(p.numel() for p in model.parameters()))
for step in range(8):
    loss = trainer.step(block).item()
    if rank == 0:
        print(f"step {step}: loss {loss:.4f}")
# the routing of one batch of router logits: slots are handed out in token order, so the same tokens
# are dropped at an overflowing expert in every run
logits = torch.randn(64, cfg.n_experts, generator=torch.Generator().manual_seed(1))
capacity = 32
weights, prob_sum, ids, slot, counts = moe_ops.route(logits, cfg.n_experts, cfg.top_k, capacity)
if rank == 0:
    print("pairs per expert", counts.tolist(), "dropped", int((slot < 0).sum()), "of", slot.numel())
