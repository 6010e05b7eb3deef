"""ZeRO-3 (FSDP x tensor parallel) MLP on a [data 2, 1, model 2] grid.

* the weights are split over BOTH grid dimensions and gathered at every use;
* checkpoint=True re-gathers them in the backward pass instead of keeping the gathered copy;
* auto_clear_buffer=False keeps the gathered copy over several micro-batches and reduce-scatters
  the accumulated gradient once (ZeRO-1 style);
* collect_state=True gives a serial PyTorch state dict on worker 0, which loads into torch.nn.Linear."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 1, 2])
from distdl_b200.nn import DistributedLinearAllGatherZero, DistributedLinearReduceScatterZero  # noqa: E402

up = DistributedLinearAllGatherZero(P, 16, 64, checkpoint=True, collect_state=True)
down = DistributedLinearReduceScatterZero(P, 64, 16, checkpoint=True, collect_state=True)
x = torch.randn(3, 5, 8, requires_grad=True)                      # [batch / 2, sequence, features / 2]
y = down(torch.relu(up(x)))
y.sum().backward()
say(P_world, "weight shards", tuple(up.weight.shape), tuple(down.weight.shape), "-> y", tuple(y.shape))

acc = DistributedLinearAllGatherZero(P, 16, 64, auto_clear_buffer=False)
for _ in range(4):                                                # four micro-batches, one reduce-scatter
    acc(torch.randn(3, 5, 8)).sum().backward()
acc.clear_weight_buffer()
say(P_world, "accumulated gradient shard", tuple(acc.weight.grad.shape))

sd = up.state_dict()
if rank == 0:
    serial = torch.nn.Linear(16, 64)
    serial.load_state_dict(sd)
    print("serial layer loaded from the gathered state:", serial)
