"""Megatron-style block: column-parallel then row-parallel linear layers with
sequence parallelism and ZeRO-3 sharding on a D=2 x M=2 grid; the state dict is
gathered in the serial torch layout on worker 0."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P_feat, P_seq = cart(P_world, [0, 1, 2, 3], [2, 1, 2]), cart(P_world, [0, 1, 2, 3], [2, 2, 1])
from distdl_b200.nn import DistributedLinearAllGatherZero, DistributedLinearReduceScatterZero  # noqa: E402

up = DistributedLinearAllGatherZero(P_feat, 16, 64, P_x=P_seq, collect_state=True)
down = DistributedLinearReduceScatterZero(P_feat, 64, 16, P_y=P_seq, collect_state=True)
x = torch.randn(2, 4, 16, requires_grad=True)          # [batch / D, seq / M, features]
y = down(torch.nn.functional.gelu(up(x)))
y.sum().backward()
say(P_world, "local weight shard", tuple(up.weight.shape), "output", tuple(y.shape))
sd = up.state_dict()
if rank == 0:
    print("serial layout on worker 0:", {k: tuple(v.shape) for k, v in sd.items()})
