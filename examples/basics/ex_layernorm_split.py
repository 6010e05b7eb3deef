"""LayerNorm over a feature dimension that is split across workers: every worker normalises
its own features with the statistics of the full rows (one exchange of per-row sums; on GPUs
with the native backend that exchange happens inside the norm kernel).

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/basics/ex_layernorm_split.py
"""
import torch
import torch.distributed as dist
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
world = dist.get_world_size()
P = cart(P_world, list(range(world)), [1, world])          # batch x features: features split over everyone
from distdl_b200.nn import DistributedLayerNorm  # noqa: E402

D = 6 * world + 1                                          # uneven on purpose: shards of 7, 6, 6, ...
ln = DistributedLayerNorm(P, D)
torch.manual_seed(0)
full = torch.randn(5, D)
sizes = [D // world + (1 if i < D % world else 0) for i in range(world)]
lo = sum(sizes[:rank])
x = full[:, lo:lo + sizes[rank]].clone().requires_grad_()
y = ln(x)
ref = torch.nn.functional.layer_norm(full, (D,))
say(P_world, "local features", tuple(x.shape), "max |y - serial|", float((y.detach() - ref[:, lo:lo + sizes[rank]]).abs().max()))
