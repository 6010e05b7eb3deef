"""Expert-parallel MLP on routed tokens [expert, capacity, sequence, features]: experts split over
E = 2 workers, features over M = 2 (tensor parallelism inside an expert); column-parallel
(all-gather) layer, activation, row-parallel (reduce-scatter) layer.  Routing itself (top-k gate,
dispatch, combine) is in distdl_b200.models.moe."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 1, 1, 2])                     # [E, N (ZeRO / capacity), 1, M]
from distdl_b200.nn import DistributedExpertAllGather, DistributedExpertReduceScatter  # noqa: E402

experts, capacity, seq, d_model, d_ff = 4, 6, 1, 16, 64
up = DistributedExpertAllGather(P, experts, d_model, d_ff, collect_state=True)
down = DistributedExpertReduceScatter(P, experts, d_ff, d_model, collect_state=True)
x = torch.randn(experts // 2, capacity, seq, d_model // 2, requires_grad=True)
y = down(torch.nn.functional.gelu(up(x)))
y.sum().backward()
say(P_world, "weight shards", tuple(up.weight.shape), tuple(down.weight.shape), "x", tuple(x.shape), "-> y",
    tuple(y.shape))
sd = up.state_dict()
if rank == 0:
    print("whole layer on worker 0:", {k: tuple(v.shape) for k, v in sd.items()})
