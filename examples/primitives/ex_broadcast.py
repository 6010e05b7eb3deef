"""Broadcast from a 1x2 partition onto a 2x2 partition and its adjoint (sum-reduce)."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P_x, P_y = cart(P_world, [0, 1], [1, 2]), cart(P_world, [0, 1, 2, 3], [2, 2])
from distdl_b200.nn import Broadcast  # noqa: E402
from distdl_b200.utilities.torch import zero_volume_tensor  # noqa: E402

layer = Broadcast(P_x, P_y, preserve_batch=False)
x = zero_volume_tensor()
if P_x.active:
    x = torch.full((2, 3), float(rank + 1))
x.requires_grad = True
y = layer(x)
say(P_world, "y =", y.tolist())
y.backward(torch.ones_like(y))
say(P_world, "dx =", x.grad.tolist())      # every source received the sum over its column
