"""SumReduce from a 2x2 partition onto its first row."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P_x, P_y = cart(P_world, [0, 1, 2, 3], [2, 2]), cart(P_world, [0, 1], [1, 2])
from distdl_b200.nn import SumReduce  # noqa: E402

y = SumReduce(P_x, P_y, preserve_batch=False)(torch.full((2,), float(rank + 1)))
say(P_world, "y =", y.tolist())
