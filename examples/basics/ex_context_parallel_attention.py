"""Attention over a sequence that is split across all workers, three ways: head <-> sequence
all-to-all (DistributedSelfAttention), K / V blocks around a ring (DistributedRingAttention), and the
ring on the load-balanced "zigzag" layout (worker r holds chunks r and 2 * world - 1 - r, so the causal
mask leaves every worker the same amount of work).  All reproduce serial causal attention.

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
hi = 2 * world - 1 - rank
zz = list(range(rank * 4, rank * 4 + 4)) + list(range(hi * 4, hi * 4 + 4))           # two chunks of 4 tokens
zig = DistributedRingAttention(P_seq, causal=True, zigzag=True)(Q[:, zz].contiguous(), K[:, zz].contiguous(),
                                                                V[:, zz].contiguous())
say(P_world, "block", rank, "max error: all-to-all", float((a2a - ref[:, sl]).abs().max()),
    "ring", float((ring - ref[:, sl]).abs().max()), "zigzag ring", float((zig - ref[:, zz]).abs().max()))
