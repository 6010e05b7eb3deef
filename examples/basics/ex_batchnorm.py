"""Batch norm of a [batch, feature, length] tensor whose batch AND feature dimensions are split
(2 x 2 workers): per-feature sums meet on one worker per feature shard, which also owns the
affine parameters and the running statistics."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 2, 1])
from distdl_b200.nn import DistributedBatchNorm  # noqa: E402

bn = DistributedBatchNorm(P, num_features=6, collect_state=True)
x = (torch.randn(4, 3, 5) * (rank + 1)).requires_grad_()       # local [batch / 2, features / 2, length]
y = bn(x)
y.square().sum().backward()
say(P_world, "gamma shard", tuple(bn.gamma.shape), "running mean", bn.running_mean.flatten().tolist())
sd = bn.state_dict()
if rank == 0:
    print("whole-layer state on worker 0:", {k: tuple(v.shape) for k, v in sd.items()})
