"""Attention over a sequence that is split across all workers, two ways: head <-> sequence
all-to-all (DistributedSelfAttention) and K / V blocks around a ring (DistributedRingAttention).
Both reproduce serial causal attention.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/basics/ex_context_parallel_attention.py
"""
import torch
import torch.distributed as dist
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
world = dist.get_world_size()
P_seq = cart(P_world, list(range(world)), [1, world, 1, 1])
from distdl_b200.nn import DistributedRingAttention, DistributedSelfAttention  # noqa: E402

b, s, heads, d = 1, 8 * world, world, 16
torch.manual_seed(0)
Q, K, V = (torch.randn(b, s, heads, d) for _ in range(3))
ref = torch.nn.functional.scaled_dot_product_attention(Q.transpose(1, 2), K.transpose(1, 2), V.transpose(1, 2),
                                                       is_causal=True).transpose(1, 2)
sl = slice(rank * 8, (rank + 1) * 8)
q, k, v = Q[:, sl].contiguous(), K[:, sl].contiguous(), V[:, sl].contiguous()
a2a = DistributedSelfAttention(P_seq, causal=True)(q, k, v)
ring = DistributedRingAttention(P_seq, causal=True)(q, k, v)
say(P_world, "block", rank, "max error: all-to-all", float((a2a - ref[:, sl]).abs().max()),
    "ring", float((ring - ref[:, sl]).abs().max()))
