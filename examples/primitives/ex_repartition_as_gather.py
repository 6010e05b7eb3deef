"""Repartition as a gather: the blocks of a 2 x 2 decomposition are assembled on worker 0."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P_x, P_root = cart(P_world, [0, 1, 2, 3], [2, 2]), cart(P_world, [0], [1, 1])
from distdl_b200.nn import Repartition  # noqa: E402

x = torch.full((2, 3), float(rank), requires_grad=True)
y = Repartition(P_x, P_root, preserve_batch=False)(x)
say(P_world, "y", y.tolist())
y.sum().backward() if y.numel() else y.backward(torch.zeros_like(y))
say(P_world, "dx", x.grad.tolist())
