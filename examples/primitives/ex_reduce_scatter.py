"""ReduceScatter along tensor dimension 0."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 2])
from distdl_b200.nn import ReduceScatter  # noqa: E402

y = ReduceScatter(P, axes_reduce_scatter=(0,))(torch.arange(6.0).reshape(6, 1) * (rank + 1))
say(P_world, "y =", y.reshape(-1).tolist())
