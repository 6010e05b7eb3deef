"""AllSumReduce along the second dimension of a 2x2 partition."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 2])
from distdl_b200.nn import AllSumReduce  # noqa: E402

y = AllSumReduce(P, axes_reduce=(1,))(torch.full((3,), float(rank + 1)))
say(P_world, "y =", y.tolist())
