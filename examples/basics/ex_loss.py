"""Distributed MSE loss: the value lives on worker 0, every worker calls backward."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 2])
from distdl_b200.nn import DistributedMSELoss  # noqa: E402

x = torch.randn(3, 4, requires_grad=True)
loss = DistributedMSELoss(P)(x, torch.zeros(3, 4))
loss.backward()
say(P_world, "loss", float(loss), "|dx|", float(x.grad.abs().sum()))
