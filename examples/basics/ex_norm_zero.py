"""LayerNorm / RMSNorm whose affine parameters are ZeRO-sharded over ALL workers and gathered on use
(the normalised dimension itself stays local: sequence parallelism)."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 2, 1])                        # [data, sequence, features]
from distdl_b200.nn import DistributedLayerNormZero, DistributedRMSNormZero  # noqa: E402

x = torch.randn(2, 5, 32, requires_grad=True)
ln, rms = DistributedLayerNormZero(P, 32, collect_state=True), DistributedRMSNormZero(P, 32, collect_state=True)
y = rms(ln(x))
y.square().sum().backward()
say(P_world, "weight shard", tuple(ln.weight.shape), "of 32; row mean", float(ln(x)[0, 0].mean()),
    "row rms", float(y[0, 0].square().mean().sqrt()))
# ZeRO-1 style: keep the gathered parameters over several micro-batches, reduce-scatter the gradient once
acc = DistributedRMSNormZero(P, 32, auto_clear_buffer=False)
for _ in range(3):
    acc(torch.randn(2, 5, 32)).sum().backward()
acc.clear_weight_buffer()
say(P_world, "accumulated gradient shard", tuple(acc.weight.grad.shape))
