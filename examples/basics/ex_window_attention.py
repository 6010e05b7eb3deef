"""Sliding-window causal attention over a sequence split across all workers: every worker fetches the last
window - 1 keys / values of its left neighbour with a halo exchange and attends locally.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/basics/ex_window_attention.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start  # noqa: E402

P_world, rank = start()
world = dist.get_world_size()
P_seq = cart(P_world, list(range(world)), [1, world, 1, 1])
from distdl_b200.nn import DistributedSlidingWindowAttention  # noqa: E402

b, s, heads, d, window = 1, 8 * world, 2, 16, 5
torch.manual_seed(0)
Q, K, V = (torch.randn(b, s, heads, d) for _ in range(3))
i, j = torch.arange(s).unsqueeze(1), torch.arange(s).unsqueeze(0)
ref = torch.nn.functional.scaled_dot_product_attention(Q.transpose(1, 2), K.transpose(1, 2), V.transpose(1, 2),
                                                       attn_mask=(j <= i) & (j > i - window)).transpose(1, 2)
sl = slice(rank * 8, (rank + 1) * 8)
out = DistributedSlidingWindowAttention(P_seq, window)(Q[:, sl].contiguous(), K[:, sl].contiguous(),
                                                        V[:, sl].contiguous())
say(P_world, "block", rank, "keys fetched from the left:", 0 if rank == 0 else window - 1,
    "max error", float((out - ref[:, sl]).abs().max()))
