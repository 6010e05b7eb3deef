"""Repartition of a 7x5 tensor from a 4x1 to a 2x2 decomposition, and back through the adjoint."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P_x, P_y = cart(P_world, [0, 1, 2, 3], [4, 1]), cart(P_world, [0, 1, 2, 3], [2, 2])
from distdl_b200.nn import Repartition  # noqa: E402
from distdl_b200.utilities.slicing import compute_start_index, compute_subshape  # noqa: E402

G = torch.arange(35.0).reshape(7, 5)
lo, sh = compute_start_index(P_x.shape, P_x.index, [7, 5]), compute_subshape(P_x.shape, P_x.index, [7, 5])
x = G[lo[0]:lo[0] + sh[0], lo[1]:lo[1] + sh[1]].clone().requires_grad_()
y = Repartition(P_x, P_y, preserve_batch=False)(x)
say(P_world, "x", x.tolist(), "-> y", y.tolist())
y.backward(torch.ones_like(y))
say(P_world, "dx", x.grad.tolist())
